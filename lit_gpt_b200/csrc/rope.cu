// Per-head preparation of projected rows before attention: an optional weighted RMS norm over the head, rotary positions on a
// run of its dimensions, and the move to where the attention reads it -- in place, to a dense buffer, or scattered into the
// rows of a cache.
//
//   z = head / sqrt(mean(head^2) + eps) * w                    (optional; statistics over the whole head, fp32)
//   (u, v) <- (u cos a - v sin a, v cos a + u sin a) * mag     for the pairs of dimensions [rot_off, rot_off + rot_dims):
//             pair i = (2 i, 2 i + 1) when interleaved, else (i, i + rot_dims / 2); a = position * freq[i] in fp32
//   the other dimensions pass unchanged.
//
// Up to three groups of heads (e.g. queries, keys, values of one fused projection) run as one launch; one CTA per (row, group).
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kHrThreads = 128, kHrMaxSegs = 3;

struct HeadSeg {
  const void* in; void* out; const void* norm_w; const float* freq; const int64_t* out_rows;
  int64_t ld_in, ld_out;
  int heads, dim, in_stride, out_stride, rot_off, rot_dims, interleaved;
  float mag;
};
struct HeadSegs { HeadSeg s[kHrMaxSegs]; };

// grid (rows, groups): the CTA of a row works out the row's cosines and sines once (they depend on the position and the pair only, not
// on the head), then its warps take the heads of the group in turn
template <typename T>
__global__ void __launch_bounds__(kHrThreads) head_rope_kernel(HeadSegs S, const int* __restrict__ row_pos, float eps) {
  extern __shared__ __align__(16) float hr_smem[];   // [rot_dims / 2] cosines, then as many sines, both times mag
  griddep_launch();
  griddep_wait();
  const HeadSeg s = S.s[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  const int64_t orow = s.out_rows ? s.out_rows[row] : row;
  if (orow < 0) return;   // a row with nowhere to go (the whole CTA leaves: no barrier is left waiting)
  const int half = s.rot_dims / 2;
  float* const cs = hr_smem;
  float* const sn = hr_smem + half;
  if (half > 0) {
    const float pos = (float)row_pos[row];
    for (int i = threadIdx.x; i < half; i += kHrThreads) {
      float a, b;
      sincosf(pos * s.freq[i], &a, &b);
      sn[i] = a * s.mag;
      cs[i] = b * s.mag;
    }
    __syncthreads();
  }
  const T* w = reinterpret_cast<const T*>(s.norm_w);
  for (int h = warp; h < s.heads; h += kHrThreads / 32) {
    const T* x = reinterpret_cast<const T*>(s.in) + row * s.ld_in + (int64_t)h * s.in_stride;
    T* o = reinterpret_cast<T*>(s.out) + orow * s.ld_out + (int64_t)h * s.out_stride;
    float rstd = 1.0f;
    if (w) {
      float ss = 0.f;
      for (int i = lane; i < s.dim; i += 32) { const float v = load_as_float(x, i); ss = fmaf(v, v, ss); }
      rstd = 1.0f / sqrtf(warp_sum(ss) / (float)s.dim + eps);   // the shuffle also orders every lane's reads before any write below
    }
    // the rotated pairs: both members are read before either is written, and no other lane touches them
    for (int i = lane; i < half; i += 32) {
      const int a = s.rot_off + (s.interleaved ? 2 * i : i), b = s.rot_off + (s.interleaved ? 2 * i + 1 : i + half);
      float u = load_as_float(x, a), v = load_as_float(x, b);
      if (w) { u = u * rstd * load_as_float(w, a); v = v * rstd * load_as_float(w, b); }
      store_from_float(o, a, u * cs[i] - v * sn[i]);
      store_from_float(o, b, v * cs[i] + u * sn[i]);
    }
    const bool moved = (const void*)o != (const void*)x;
    if (!w && !moved) continue;
    for (int i = lane; i < s.dim; i += 32) {
      if (i >= s.rot_off && i < s.rot_off + 2 * half) continue;
      float v = load_as_float(x, i);
      if (w) v = v * rstd * load_as_float(w, i);
      store_from_float(o, i, v);
    }
  }
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_head_rope(const b200_head_rope_seg* segs, int n_segs, const int32_t* row_pos, int64_t rows, float eps, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(segs && n_segs >= 1 && n_segs <= kHrMaxSegs && row_pos, "b200_head_rope: one to three groups of heads and the rows' positions");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff, "b200_head_rope: bad row count");
  HeadSegs S;
  int max_rot = 0;
  for (int i = 0; i < kHrMaxSegs; ++i) {
    const b200_head_rope_seg& a = segs[i < n_segs ? i : 0];
    B200_CHECK_ARG(a.in && a.out && a.heads > 0 && a.dim > 0, "b200_head_rope: null pointer or empty head");
    B200_CHECK_ARG(a.rot_dims >= 0 && a.rot_dims % 2 == 0 && a.rot_off >= 0 && a.rot_off + a.rot_dims <= a.dim && (a.rot_dims == 0 || a.freq),
                   "b200_head_rope: the rotated dimensions must be an even run inside the head, with their frequencies");
    S.s[i] = HeadSeg{a.in, a.out, a.norm_w, a.freq, a.out_rows, a.ld_in, a.ld_out, a.heads, a.dim, a.in_stride, a.out_stride, a.rot_off, a.rot_dims,
                     a.interleaved, a.mag};
    if (i < n_segs) max_rot = a.rot_dims > max_rot ? a.rot_dims : max_rot;
  }
  B200_CHECK_ARG(max_rot <= 8192, "b200_head_rope: at most 8192 rotated dimensions");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(head_rope_kernel<T>, dim3((unsigned)rows, (unsigned)n_segs), dim3(kHrThreads), (size_t)max_rot * sizeof(float),
                                               (cudaStream_t)stream, S, row_pos, eps)));
  return B200_OK;
}

}  // extern "C"
