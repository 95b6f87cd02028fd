// Residual update of a block whose norms work in GROUPS, with an optional weighted average over depth.
//
//   gnorm(z) : the row is cut into `groups` equal consecutive pieces; each piece is divided by its own sqrt(mean(piece^2) + eps)
//   x_out = x_in + gnorm(y) * post_w                              (fp32; without y: x_out = x_in)
//   avg   = sum_{j < m} depth_w[j] * X_j                          (optional; X_0 .. X_{m-2} are rows of `stack`, X_{m-1} = x_out)
//   act   = T(gnorm(avg, or x_out without the average) * pre_w)   (optional: the norm that feeds whatever reads the stream next)
//
// A model that averages over depth keeps every layer's own result X_j of the step in one (layers + 1, rows, d) fp32 stack; what
// a layer reads is the average its predecessor left.  One CTA per row, the row in shared memory between the passes; statistics,
// sums and the stream are fp32 whatever the matrix-product dtype T is.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kDrThreads = 128;

struct DepthArgs {
  const void* y; const void* post_w;
  const float* x_in; float* x_out;
  const float* stack; int64_t stack_stride; const void* depth_w; float* avg;
  const void* pre_w; void* act;
  int d, groups, m;
  float eps;
};

// 1 / sqrt(mean + eps) of every group of the row in `row` (shared memory) -> rs[groups]; a warp takes every fourth group
__device__ __forceinline__ void group_rstd(const float* row, float* rs, int d, int groups, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, per = d / groups;
  __syncthreads();   // the row is complete, rs is no longer read
  for (int g = warp; g < groups; g += kDrThreads / 32) {
    const float* p = row + (int64_t)g * per;
    float ss = 0.f;
    for (int i = lane; i < per; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) rs[g] = 1.0f / sqrtf(ss / (float)per + eps);
  }
  __syncthreads();
}

// V: elements per access (4 when the row length, every base and every row start allow 16-byte accesses of fp32 / 8-byte of bf16)
template <typename T, int V>
__device__ __forceinline__ void ldv(const T* p, int64_t i, float (&f)[V]) {
  if constexpr (V == 1) {
    f[0] = load_as_float(p, i);
  } else if constexpr (sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p + i);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(p + i);
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  }
}
template <typename T, int V>
__device__ __forceinline__ void stv(T* p, int64_t i, const float (&f)[V]) {
  if constexpr (V == 1) {
    store_from_float(p, i, f[0]);
  } else if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p + i) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    *reinterpret_cast<uint2*>(p + i) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kDrThreads) depth_residual_kernel(DepthArgs A) {
  extern __shared__ __align__(16) float dr_smem[];   // [d] the row, then [groups] reciprocal deviations
  griddep_launch();
  griddep_wait();
  const int d = A.d, groups = A.groups, per = d / groups;
  float* const row = dr_smem;
  float* const rs = dr_smem + ((d + 3) & ~3);
  const int64_t base = (int64_t)blockIdx.x * d;
  const T* y = reinterpret_cast<const T*>(A.y);
  const T* pw = reinterpret_cast<const T*>(A.post_w);
  const T* dw = reinterpret_cast<const T*>(A.depth_w);
  const T* nw = reinterpret_cast<const T*>(A.pre_w);
  // every thread touches the same elements in every pass, so the row needs barriers only around the group statistics
  if (y) {
    for (int i = threadIdx.x * V; i < d; i += kDrThreads * V) {
      float v[V];
      ldv<T, V>(y, base + i, v);
#pragma unroll
      for (int j = 0; j < V; ++j) row[i + j] = v[j];
    }
    group_rstd(row, rs, d, groups, A.eps);
  }
  for (int i = threadIdx.x * V; i < d; i += kDrThreads * V) {
    float xv[V];
    ldv<float, V>(A.x_in, base + i, xv);
    if (y) {
      float g[V];
      ldv<T, V>(pw, i, g);
      const float r = rs[i / per];   // V divides the group length when V > 1
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] = xv[j] + row[i + j] * r * g[j];
    }
    if (y || A.x_out != A.x_in) stv<float, V>(A.x_out, base + i, xv);
    if (A.avg) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int l = 0; l + 1 < A.m; ++l) {
        const float wl = load_as_float(dw, l);
        float s[V];
        ldv<float, V>(A.stack + (int64_t)l * A.stack_stride, base + i, s);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = fmaf(wl, s[j], acc[j]);
      }
      const float wl = load_as_float(dw, A.m - 1);
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] = fmaf(wl, xv[j], acc[j]);
      stv<float, V>(A.avg, base + i, xv);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) row[i + j] = xv[j];
  }
  if (!nw) return;
  group_rstd(row, rs, d, groups, A.eps);
  T* ar = reinterpret_cast<T*>(A.act);
  for (int i = threadIdx.x * V; i < d; i += kDrThreads * V) {
    float g[V], o[V];
    ldv<T, V>(nw, i, g);
    const float r = rs[i / per];
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = row[i + j] * r * g[j];
    stv<T, V>(ar, base + i, o);
  }
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_depth_residual(const b200_depth_residual_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->x_in && a->x_out, "b200_depth_residual: null pointer");
  B200_CHECK_ARG(!a->y || a->post_w, "b200_depth_residual: a branch needs its norm weight");
  B200_CHECK_ARG(!a->pre_w || a->act, "b200_depth_residual: the next norm needs somewhere to go");
  B200_CHECK_ARG(!a->avg || (a->depth_w && a->m >= 1 && (a->m == 1 || a->stack)), "b200_depth_residual: the average needs its weights and the earlier results");
  B200_CHECK_ARG(a->rows > 0 && a->rows <= 0x7fffffff && a->d > 0 && a->groups > 0 && a->d % a->groups == 0, "b200_depth_residual: bad shape");
  const size_t smem = ((size_t)((a->d + 3) & ~3) + (size_t)a->groups) * sizeof(float);
  B200_CHECK_ARG(smem <= 160 * 1024, "b200_depth_residual: rows of %d numbers do not fit shared memory", a->d);
  const DepthArgs A{a->y, a->post_w, a->x_in, a->x_out, a->stack, a->stack_stride, a->depth_w, a->avg, a->pre_w, a->act, a->d, a->groups, a->m, a->eps};
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a->y) | reinterpret_cast<uintptr_t>(a->post_w) | reinterpret_cast<uintptr_t>(a->x_in) |
                         reinterpret_cast<uintptr_t>(a->x_out) | reinterpret_cast<uintptr_t>(a->stack) | reinterpret_cast<uintptr_t>(a->avg) |
                         reinterpret_cast<uintptr_t>(a->pre_w) | reinterpret_cast<uintptr_t>(a->act);
  const bool vec = (a->d / a->groups) % 4 == 0 && (ptrs & 15) == 0 && (a->stack_stride & 3) == 0;
  B200_FLOAT_TYPES(a->dtype, T, {
    static PerDeviceOnce once;
    if (smem > 48 * 1024 && once.need()) {
      B200_CUDA(cudaFuncSetAttribute(depth_residual_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      B200_CUDA(cudaFuncSetAttribute(depth_residual_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      once.done();
    }
    if (vec) B200_CUDA(launch(depth_residual_kernel<T, 4>, dim3((unsigned)a->rows), dim3(kDrThreads), smem, (cudaStream_t)stream, A));
    else B200_CUDA(launch(depth_residual_kernel<T, 1>, dim3((unsigned)a->rows), dim3(kDrThreads), smem, (cudaStream_t)stream, A));
  });
  return B200_OK;
}

}  // extern "C"
