// Sparse mixture of experts: a router (sigmoid or softmax scores, optional selection bias, group-limited choice) and the
// expert feed-forward over stacked expert weights: y = W_down relu(W_up x)^2 with W_up (E, ff, d), or the gated form
// y = W_down (silu(W_gate x) * (W_up x)) with the gate and up rows stacked as (E, 2 ff, d); W_down (E, d, ff).
//
//  * b200_moe_route: logits, scores, choice and weights in fp32, one CTA per token.
//  * b200_moe_plan: counting sort of the (token, choice) pairs by expert -> contiguous row ranges per expert.
//  * b200_moe_gemm: grouped matrix product over those ranges (one launch for all experts, no host round trip), any
//    sizes, bf16 or fp32 operands, fp32 accumulation; optional gather of the input rows and relu^2 epilogue.
//  * b200_moe_gemv_up / b200_moe_gemv_down: the same two products for a handful of tokens (decode), where every chosen
//    expert's weights are streamed exactly once and the weighted sum over the choices is part of the second kernel.
//  * b200_moe_combine: out[t] = sum_k weight[t, k] * y[slot(t, k)], in the fixed order of k (deterministic).
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kRtThreads = 256;

// argmax over v[0..n) by the 32 lanes of a warp: largest value, lowest index among equals; every lane gets the index
__device__ __forceinline__ int warp_argmax(const float* v, int n, int lane) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lane; i < n; i += 32) {
    const float x = v[i];
    if (bi == 0x7fffffff || x > best) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
  }
  return bi;
}

template <typename T>
__global__ void __launch_bounds__(kRtThreads) moe_route_kernel(const T* __restrict__ x, const T* __restrict__ w_router,
                                                                const T* __restrict__ correction, int* __restrict__ ids,
                                                                float* __restrict__ wts, int d, int n_expert, int top, int n_group,
                                                                int keep, int flags) {
  extern __shared__ float rt_smem[];
  griddep_launch();
  griddep_wait();
  float* const score = rt_smem;               // [E] sigmoid(z)
  float* const choice = score + n_expert;     // [E] score + correction, -inf once excluded or taken
  float* const grank = choice + n_expert;     // [G]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = blockIdx.x;
  const T* xr = x + t * d;
  for (int e = warp; e < n_expert; e += kRtThreads / 32) {
    const float z = warp_dot(xr, w_router + (int64_t)e * d, d, lane);
    if (lane == 0) {
      const float corr = correction ? load_as_float(correction, e) : 0.f;
      const float zz = (flags & B200_ROUTE_BIAS) ? z + corr : z;     // a bias is part of the logit; a correction only steers the choice
      const float s = (flags & (B200_ROUTE_SOFTMAX | B200_ROUTE_TOPK_SOFTMAX)) ? zz : 1.0f / (1.0f + expf(-zz));
      score[e] = s;
      choice[e] = (flags & B200_ROUTE_BIAS) ? s : s + corr;
    }
  }
  __syncthreads();
  if (flags & B200_ROUTE_SOFTMAX) {   // scores = softmax over ALL experts, before any group is excluded
    if (warp == 0) {
      float mx = -INFINITY;
      for (int e = lane; e < n_expert; e += 32) mx = fmaxf(mx, score[e]);
      mx = warp_max(mx);
      float sum = 0.f;
      for (int e = lane; e < n_expert; e += 32) sum += expf(score[e] - mx);
      sum = warp_sum(sum);
      for (int e = lane; e < n_expert; e += 32) {
        const float s = expf(score[e] - mx) / sum;
        score[e] = s;
        choice[e] = s + (correction && !(flags & B200_ROUTE_BIAS) ? load_as_float(correction, e) : 0.f);
      }
    }
    __syncthreads();
  }
  const int per = n_expert / n_group;
  for (int g = tid; g < n_group; g += kRtThreads) {   // a group's rank: the sum of its two largest choice scores, or the largest
    float a = -INFINITY, b = -INFINITY;
    for (int i = 0; i < per; ++i) {
      const float c = choice[g * per + i];
      if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
    }
    grank[g] = (per > 1 && !(flags & B200_ROUTE_GROUP_MAX)) ? a + b : a;
  }
  __syncthreads();
  if (warp != 0) return;
  if (keep < n_group) {
    // take the `keep` best groups (marked by a rank of -inf), then exclude the experts of all others
    for (int k = 0; k < keep; ++k) {
      const int g = warp_argmax(grank, n_group, lane);
      __syncwarp();
      if (lane == 0) grank[g] = -INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_expert; e += 32)
      if (grank[e / per] != -INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    const int e = warp_argmax(choice, n_expert, lane);
    __syncwarp();
    if (lane == 0) {
      ids[t * top + k] = e;
      wts[t * top + k] = score[e];
      choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  if ((flags & B200_ROUTE_TOPK_SOFTMAX) && lane == 0) {   // weights = softmax among those `top` logits
    float mx = -INFINITY, sum = 0.f;
    for (int k = 0; k < top; ++k) mx = fmaxf(mx, score[ids[t * top + k]]);
    for (int k = 0; k < top; ++k) sum += expf(score[ids[t * top + k]] - mx);
    for (int k = 0; k < top; ++k) wts[t * top + k] = expf(score[ids[t * top + k]] - mx) / sum;
  }
}

// One CTA.  counts -> expert_off[E + 1] (rows), tile_off[E + 1] (row tiles of `tile_rows`), slot_token[slot] = token,
// slot_of[t * top + k] = slot.
__global__ void __launch_bounds__(256) moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int top, int n_expert, int tile_rows,
                                                       int* __restrict__ expert_off, int* __restrict__ tile_off,
                                                       int* __restrict__ slot_token, int* __restrict__ slot_of) {
  extern __shared__ int pl_smem[];   // [E] counts, then cursors; [E + 1] offsets
  griddep_launch();
  griddep_wait();
  int* const cnt = pl_smem;
  int* const off = cnt + n_expert;
  for (int e = threadIdx.x; e < n_expert; e += 256) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += 256) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < n_expert; ++e) {
      off[e] = rows;
      expert_off[e] = rows;
      tile_off[e] = tiles;
      rows += cnt[e];
      tiles += (cnt[e] + tile_rows - 1) / tile_rows;
      cnt[e] = 0;
    }
    off[n_expert] = rows;
    expert_off[n_expert] = rows;
    tile_off[n_expert] = tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += 256) {
    const int e = ids[i];
    const int slot = off[e] + atomicAdd(&cnt[e], 1);
    slot_token[slot] = i / top;
    slot_of[i] = slot;
  }
}

// Grouped product: for expert e and its rows [expert_off[e], expert_off[e + 1]):
//   C[row, n] = act( sum_k A[src(row), k] * W[e][n, k] ),  src(row) = row_src ? row_src[row] : row.
// 64 x 64 tile per CTA, 32-deep k steps, 4 x 4 register tile per thread, operands converted to fp32 in shared memory.
constexpr int kGmBM = 64, kGmBN = 64, kGmBK = 32, kGmPitch = 36, kGmThreads = 256;

template <typename T, bool SQRELU>
__global__ void __launch_bounds__(kGmThreads) moe_gemm_kernel(const T* __restrict__ A, int64_t lda, const int* __restrict__ row_src,
                                                               const T* __restrict__ W, T* __restrict__ C, int64_t ldc,
                                                               const int* __restrict__ expert_off, const int* __restrict__ tile_off,
                                                               int n_expert, int N, int K) {
  __shared__ __align__(16) float As[kGmBM * kGmPitch];
  __shared__ __align__(16) float Ws[kGmBN * kGmPitch];
  __shared__ int s_src[kGmBM];
  griddep_launch();
  griddep_wait();
  const int tile = blockIdx.x;
  if (tile >= tile_off[n_expert]) return;
  int e = 0;
  while (tile >= tile_off[e + 1]) ++e;     // E is small; every thread walks the same way
  const int row0 = expert_off[e] + (tile - tile_off[e]) * kGmBM;
  const int rows = min(kGmBM, expert_off[e + 1] - row0);
  const int n0 = blockIdx.y * kGmBN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < kGmBM) s_src[tid] = tid < rows ? (row_src ? row_src[row0 + tid] : row0 + tid) : -1;
  const T* We = W + (int64_t)e * N * K;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  __syncthreads();
  const int lr = tid >> 2, lk = (tid & 3) * 8;   // this thread loads 8 consecutive k of one row of each operand
  for (int k0 = 0; k0 < K; k0 += kGmBK) {
    const int src = s_src[lr];
    const int wn = n0 + lr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kk = k0 + lk + i;
      As[lr * kGmPitch + lk + i] = (src >= 0 && kk < K) ? load_as_float(A, (int64_t)src * lda + kk) : 0.f;
      Ws[lr * kGmPitch + lk + i] = (wn < N && kk < K) ? load_as_float(We, (int64_t)wn * K + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGmBK; kk += 4) {
      float4 av[4], wv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) av[a] = *reinterpret_cast<const float4*>(As + (ty + 16 * a) * kGmPitch + kk);
#pragma unroll
      for (int b = 0; b < 4; ++b) wv[b] = *reinterpret_cast<const float4*>(Ws + (tx + 16 * b) * kGmPitch + kk);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          acc[a][b] = fmaf(av[a].x, wv[b].x, acc[a][b]);
          acc[a][b] = fmaf(av[a].y, wv[b].y, acc[a][b]);
          acc[a][b] = fmaf(av[a].z, wv[b].z, acc[a][b]);
          acc[a][b] = fmaf(av[a].w, wv[b].w, acc[a][b]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = ty + 16 * a;
    if (r >= rows) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int n = n0 + tx + 16 * b;
      if (n >= N) continue;
      float v = acc[a][b];
      if (SQRELU) { v = fmaxf(v, 0.f); v *= v; }
      store_from_float(C, (int64_t)(row0 + r) * ldc + n, v);
    }
  }
}

// decode: hidden[p, f] = relu(W_up[ids[p]][f, :] . x[p / top, :])^2 for the pair p = t * top + k; one warp per f.
// GATED: W_up holds 2 ff rows per expert and hidden[p, f] = silu(row f . x) * (row ff + f . x).
// limit > 0: the clamped form g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_gemv_up_kernel(const T* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ w_up,
                                                          T* __restrict__ hidden, int top, int d, int ff, float limit, float alpha) {
  griddep_launch();
  griddep_wait();
  const int p = blockIdx.y, lane = threadIdx.x & 31;
  const int f = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (f >= ff) return;
  const T* xr = x + (int64_t)(p / top) * d;
  if (GATED) {
    const T* wg = w_up + ((int64_t)ids[p] * 2 * ff + f) * d;
    const float gate = warp_dot(wg, xr, d, lane), up = warp_dot(wg + (int64_t)ff * d, xr, d, lane);
    if (lane == 0) {   // both products take the matrix-product dtype before the activation, as in the grouped path
      T gr, ur;
      store_from_float(&gr, 0, gate);
      store_from_float(&ur, 0, up);
      float gz = load_as_float(&gr, 0), uz = load_as_float(&ur, 0);
      if (limit > 0.f) {
        gz = fminf(gz, limit);
        uz = fminf(fmaxf(uz, -limit), limit);
        store_from_float(hidden, (int64_t)p * ff + f, gz / (1.0f + expf(-alpha * gz)) * (uz + 1.0f));
      } else {
        store_from_float(hidden, (int64_t)p * ff + f, gz / (1.0f + expf(-gz)) * uz);
      }
    }
    return;
  }
  const T* wr = w_up + ((int64_t)ids[p] * ff + f) * d;
  float acc = warp_dot(wr, xr, d, lane);
  if (lane == 0) {
    acc = fmaxf(acc, 0.f);
    store_from_float(hidden, (int64_t)p * ff + f, acc * acc);
  }
}

// decode: out[t, c] = sum_k wts[t, k] * T(W_down[ids[t, k]][c, :] . hidden[t * top + k, :]); one warp per c
template <typename T>
__global__ void __launch_bounds__(256) moe_gemv_down_kernel(const T* __restrict__ hidden, const int* __restrict__ ids,
                                                            const float* __restrict__ wts, const T* __restrict__ w_down,
                                                            T* __restrict__ out, int top, int d, int ff) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (c >= d) return;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    const int p = t * top + k;
    const T* hr = hidden + (int64_t)p * ff;
    const T* wr = w_down + ((int64_t)ids[p] * d + c) * ff;
    const float acc = warp_dot(wr, hr, ff, lane);
    T rounded;   // the expert's output takes the matrix-product dtype before it is weighted, as in the grouped path
    store_from_float(&rounded, 0, acc);
    total = fmaf(wts[p], load_as_float(&rounded, 0), total);
  }
  if (lane == 0) store_from_float(out, (int64_t)t * d + c, total);
}

template <typename T>
__global__ void __launch_bounds__(128) moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ slot_of,
                                                          const float* __restrict__ wts, T* __restrict__ out, int top, int d) {
  griddep_launch();
  griddep_wait();
  const int64_t t = blockIdx.x;
  if (vec8_ok(d, y, out)) {
    for (int c = threadIdx.x * 8; c < d; c += 128 * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < top; ++k) {
        float v[8];
        load8(y + (int64_t)slot_of[t * top + k] * d + c, v);
        const float w = wts[t * top + k];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, v[j], acc[j]);
      }
      store8(out + t * d + c, acc);
    }
    return;
  }
  for (int c = threadIdx.x; c < d; c += 128) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(wts[t * top + k], load_as_float(y, (int64_t)slot_of[t * top + k] * d + c), acc);
    store_from_float(out, t * d + c, acc);
  }
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_moe_route(const void* x, const void* w_router, const void* correction, int32_t* ids, float* weights, int64_t tokens, int d,
                   int n_expert, int top, int n_group, int keep, int flags, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(x && w_router && ids && weights, "b200_moe_route: null pointer");
  B200_CHECK_ARG(tokens > 0 && tokens <= 0x7fffffff && d > 0 && n_expert > 0 && top > 0 && top <= n_expert, "b200_moe_route: bad shape");
  B200_CHECK_ARG(n_group > 0 && n_expert % n_group == 0 && keep > 0 && keep <= n_group, "b200_moe_route: groups must divide the experts");
  B200_CHECK_ARG((int64_t)keep * (n_expert / n_group) >= top, "b200_moe_route: the kept groups hold fewer experts than are chosen");
  const size_t smem = (size_t)(2 * n_expert + n_group) * sizeof(float);
  B200_CHECK_ARG(smem <= 48 * 1024, "b200_moe_route: too many experts");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(moe_route_kernel<T>, dim3((unsigned)tokens), dim3(kRtThreads), smem, (cudaStream_t)stream, (const T*)x,
                                               (const T*)w_router, (const T*)correction, ids, weights, d, n_expert, top, n_group, keep, flags)));
  return B200_OK;
}

int b200_moe_plan(const int32_t* ids, int64_t tokens, int top, int n_expert, int32_t* expert_off, int32_t* tile_off, int32_t* slot_token,
                  int32_t* slot_of, b200_stream_t stream) {
  B200_CHECK_ARG(ids && expert_off && tile_off && slot_token && slot_of, "b200_moe_plan: null pointer");
  B200_CHECK_ARG(tokens > 0 && tokens * top <= 0x7fffffff && n_expert > 0 && n_expert <= 4096, "b200_moe_plan: bad shape");
  B200_CUDA(launch(moe_plan_kernel, dim3(1), dim3(256), (size_t)(2 * n_expert + 1) * sizeof(int), (cudaStream_t)stream, ids, (int)(tokens * top), top,
                   n_expert, kGmBM, expert_off, tile_off, slot_token, slot_of));
  return B200_OK;
}

int b200_moe_gemm(const void* a, int64_t lda, const int32_t* row_src, const void* w, void* c, int64_t ldc, const int32_t* expert_off,
                  const int32_t* tile_off, int64_t rows, int n_expert, int n, int k, int sqrelu, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(a && w && c && expert_off && tile_off, "b200_moe_gemm: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && k > 0 && n_expert > 0, "b200_moe_gemm: bad shape");
  const int64_t tiles = (rows + kGmBM - 1) / kGmBM + n_expert;   // upper bound; CTAs past the planned count return at once
  B200_CHECK_ARG(tiles <= 0x7fffffff && (n + kGmBN - 1) / kGmBN <= 65535, "b200_moe_gemm: too large");
  const dim3 grid((unsigned)tiles, (unsigned)((n + kGmBN - 1) / kGmBN)), block(kGmThreads);
  cudaStream_t st = (cudaStream_t)stream;
  if (sqrelu)
    B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(moe_gemm_kernel<T, true>, grid, block, 0, st, (const T*)a, lda, row_src, (const T*)w, (T*)c, ldc,
                                                 expert_off, tile_off, n_expert, n, k)));
  else
    B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(moe_gemm_kernel<T, false>, grid, block, 0, st, (const T*)a, lda, row_src, (const T*)w, (T*)c, ldc,
                                                 expert_off, tile_off, n_expert, n, k)));
  return B200_OK;
}

int b200_moe_gemv(const void* x, const int32_t* ids, const float* weights, const void* w_up, const void* w_down, void* hidden, void* out,
                  int64_t tokens, int top, int d, int ff, int gated, float limit, float alpha, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(x && ids && weights && w_up && w_down && hidden && out, "b200_moe_gemv: null pointer");
  B200_CHECK_ARG(gated >= 0 && gated <= 2 && (gated != 2 || limit > 0.f), "b200_moe_gemv: gated is 0 (relu^2), 1 (silu gate) or 2 (clamped gate, limit > 0)");
  if (gated != 2) limit = 0.f;
  B200_CHECK_ARG(tokens > 0 && tokens * top <= 65535 && d > 0 && ff > 0, "b200_moe_gemv: bad shape");
  cudaStream_t st = (cudaStream_t)stream;
  B200_FLOAT_TYPES(dtype, T, {
    if (gated)
      B200_CUDA(launch(moe_gemv_up_kernel<T, true>, dim3((unsigned)((ff + 7) / 8), (unsigned)(tokens * top)), dim3(256), 0, st, (const T*)x, ids,
                       (const T*)w_up, (T*)hidden, top, d, ff, limit, alpha));
    else
      B200_CUDA(launch(moe_gemv_up_kernel<T, false>, dim3((unsigned)((ff + 7) / 8), (unsigned)(tokens * top)), dim3(256), 0, st, (const T*)x, ids,
                       (const T*)w_up, (T*)hidden, top, d, ff, limit, alpha));
    B200_CUDA(launch(moe_gemv_down_kernel<T>, dim3((unsigned)((d + 7) / 8), (unsigned)tokens), dim3(256), 0, st, (const T*)hidden, ids, weights,
                     (const T*)w_down, (T*)out, top, d, ff));
  });
  return B200_OK;
}

int b200_moe_combine(const void* y, const int32_t* slot_of, const float* weights, void* out, int64_t tokens, int top, int d, int dtype,
                     b200_stream_t stream) {
  B200_CHECK_ARG(y && slot_of && weights && out && tokens > 0 && tokens <= 0x7fffffff && top > 0 && d > 0, "b200_moe_combine: bad argument");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(moe_combine_kernel<T>, dim3((unsigned)tokens), dim3(128), 0, (cudaStream_t)stream, (const T*)y, slot_of,
                                               weights, (T*)out, top, d)));
  return B200_OK;
}

}  // extern "C"
