// Latent attention: attention whose keys and values are up-projections of one small cached vector per position
// (the "latent" c, r numbers).  Per head h: k = W_uk[h] c, v = W_uv[h] c, score = (q_h . k) * scale, causal softmax in fp32.
// Only c is cached, so a layer may attend over ANOTHER layer's latents with its own W_uk / W_uv.
// Optional parts, each a parameter: a second key part shared by all heads (e.g. rotated dimensions: the query head is then
// [dk unrotated | dk2 shared-part] numbers and the cache row [c | shared part], rotated before it is stored), a per-head sink
// logit that joins the softmax denominator only, and a sigmoid output gate per head or per output number.
//
// Two kernels families:
//  * prefill (many query rows per sequence): K and V of the context are expanded by a matrix product outside; the kernel
//    here is a tiled flash attention over ragged sequences with separate query-key and value sizes, any sizes, operands
//    bf16 or fp32, all arithmetic fp32 (online softmax with a running maximum).
//  * decode (one query row per sequence): the up-projections are absorbed -- q'_h = W_uk[h]^T q_h (r numbers), scores are
//    q'_h . c_j over the cached latents, the probabilities average the latents themselves, and W_uv[h] is applied once to
//    that average.  Work per cached position is 2 r MACs per head instead of re-expanding dk + dv numbers; the context is
//    split over CTAs (split-K) and a last kernel merges the splits and applies W_uv.  For bf16 the split runs on the
//    tensor cores with sixteen heads as the rows of one tile; fp32 models and odd latent sizes take the any-size kernel.
#include <algorithm>
#include <type_traits>

#include "mma_tile.cuh"

namespace b200 {

namespace {

// ---------------------------------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------------------------------
constexpr int kLpBM = 64, kLpBN = 64, kLpDV = 128, kLpThreads = 256;

// row pitch (floats) for a tile whose rows are read as float4 by lanes one row apart: a multiple of 4 with pitch/4 odd, so
// that the eight lanes of a quarter-warp hit eight different 16-byte bank groups
__host__ __device__ inline int conflict_free_pitch(int d) {
  int p = (d + 3) & ~3;
  if (((p >> 2) & 1) == 0) p += 4;
  return p;
}

// seq: {first query row in the packed batch, number of query rows, position of the first query row,
//       row of position 0 of this sequence in the expanded K / V buffers}
template <typename T>
__global__ void __launch_bounds__(kLpThreads) latent_prefill_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k,
                                                                     int64_t ldk, const T* __restrict__ v, int64_t ldv,
                                                                     const int4* __restrict__ seqs, T* __restrict__ out, int64_t ldo,
                                                                     int n_head, int dk, int dv, float scale_log2,
                                                                     const T* __restrict__ k2, int64_t ldk2, int dk2,
                                                                     const T* __restrict__ sink, const T* __restrict__ gate, int64_t ldg,
                                                                     int gate_mode) {
  // dk counts the whole query head; its last dk2 numbers meet the shared key part k2 (one per position, the same for every head)
  extern __shared__ __align__(16) float lp_smem[];
  griddep_launch();
  griddep_wait();
  const int4 sq = seqs[blockIdx.z];
  const int qstart = sq.x, qlen = sq.y, pos0 = sq.z, kvstart = sq.w;
  const int r0 = (int)blockIdx.x * kLpBM;
  if (r0 >= qlen) return;
  const int nchunk = (dv + kLpDV - 1) / kLpDV;
  const int h = (int)blockIdx.y / nchunk, c0 = ((int)blockIdx.y % nchunk) * kLpDV;
  const int dvc = min(kLpDV, dv - c0);
  const int dkp = conflict_free_pitch(dk), dk1 = dk - dk2;
  constexpr int PP = kLpBN + 4;                       // pitch of the probability tile (68: 17 is odd)
  float* const Qs = lp_smem;                          // [64][dkp]
  float* const Ks = Qs + kLpBM * dkp;                 // [64][dkp]
  float* const Vs = Ks + kLpBN * dkp;                 // [64][128]
  float* const Ps = Vs + kLpBN * kLpDV;               // [64][68]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  // Q tile, pre-multiplied by scale * log2(e); rows past the sequence and the padding columns are zero
  for (int idx = tid; idx < kLpBM * dkp; idx += kLpThreads) {
    const int i = idx / dkp, d = idx - i * dkp;
    float val = 0.f;
    if (r0 + i < qlen && d < dk) val = load_as_float(q, (int64_t)(qstart + r0 + i) * ldq + (int64_t)h * dk + d) * scale_log2;
    Qs[idx] = val;
  }
  const int last_row = min(r0 + kLpBM, qlen) - 1;
  const int n_keys = pos0 + last_row + 1;             // keys 0 .. position of the tile's last valid row

  float o[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) o[a][b] = 0.f;
  float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l_run[4] = {0.f, 0.f, 0.f, 0.f};
  int lim[4];                                         // last visible key of each of this thread's rows (-1: no row)
#pragma unroll
  for (int a = 0; a < 4; ++a) lim[a] = (r0 + ty + 16 * a < qlen) ? pos0 + r0 + ty + 16 * a : -1;

  for (int j0 = 0; j0 < n_keys; j0 += kLpBN) {
    __syncthreads();                                  // previous tile fully consumed (and Q visible on the first pass)
    for (int idx = tid; idx < kLpBN * dkp; idx += kLpThreads) {
      const int j = idx / dkp, d = idx - j * dkp;
      float val = 0.f;
      if (j0 + j < n_keys && d < dk)
        val = d < dk1 ? load_as_float(k, (int64_t)(kvstart + j0 + j) * ldk + (int64_t)h * dk1 + d)
                      : load_as_float(k2, (int64_t)(kvstart + j0 + j) * ldk2 + (d - dk1));
      Ks[idx] = val;
    }
    for (int idx = tid; idx < kLpBN * kLpDV; idx += kLpThreads) {
      const int j = idx / kLpDV, c = idx - j * kLpDV;
      float val = 0.f;
      if (j0 + j < n_keys && c < dvc) val = load_as_float(v, (int64_t)(kvstart + j0 + j) * ldv + (int64_t)h * dv + c0 + c);
      Vs[idx] = val;
    }
    __syncthreads();

    // S = Q K^T for rows ty + 16 a, keys tx + 16 b
    float s[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
    for (int d = 0; d < dkp; d += 4) {
      float4 qa[4], kb[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) qa[a] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * a) * dkp + d);
#pragma unroll
      for (int b = 0; b < 4; ++b) kb[b] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * b) * dkp + d);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          s[a][b] = fmaf(qa[a].x, kb[b].x, s[a][b]);
          s[a][b] = fmaf(qa[a].y, kb[b].y, s[a][b]);
          s[a][b] = fmaf(qa[a].z, kb[b].z, s[a][b]);
          s[a][b] = fmaf(qa[a].w, kb[b].w, s[a][b]);
        }
    }
    // causal mask, running maximum, probabilities
    float alpha[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float mx = -INFINITY;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (j0 + tx + 16 * b > lim[a]) s[a][b] = -INFINITY;
        mx = fmaxf(mx, s[a][b]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[a], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[a] = exp2f(m_run[a] - m_safe);            // exp2(-inf) = 0 on the first tile
      float ps = 0.f;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float p = exp2f(s[a][b] - m_safe);
        ps += p;
        Ps[(ty + 16 * a) * PP + tx + 16 * b] = p;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l_run[a] = l_run[a] * alpha[a] + ps;
      m_run[a] = m_new;
#pragma unroll
      for (int b = 0; b < 8; ++b) o[a][b] *= alpha[a];
    }
    __syncthreads();
    // O += P V for rows ty + 16 a, value columns 4 tx .. 4 tx + 3 and 64 + 4 tx .. 64 + 4 tx + 3
    for (int j = 0; j < kLpBN; j += 4) {
      float4 pa[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) pa[a] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * a) * PP + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 v0 = *reinterpret_cast<const float4*>(Vs + (j + jj) * kLpDV + 4 * tx);
        const float4 v1 = *reinterpret_cast<const float4*>(Vs + (j + jj) * kLpDV + 64 + 4 * tx);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float p = jj == 0 ? pa[a].x : jj == 1 ? pa[a].y : jj == 2 ? pa[a].z : pa[a].w;
          o[a][0] = fmaf(p, v0.x, o[a][0]); o[a][1] = fmaf(p, v0.y, o[a][1]);
          o[a][2] = fmaf(p, v0.z, o[a][2]); o[a][3] = fmaf(p, v0.w, o[a][3]);
          o[a][4] = fmaf(p, v1.x, o[a][4]); o[a][5] = fmaf(p, v1.y, o[a][5]);
          o[a][6] = fmaf(p, v1.z, o[a][6]); o[a][7] = fmaf(p, v1.w, o[a][7]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = r0 + ty + 16 * a;
    if (i >= qlen) continue;
    float den = l_run[a];
    if (sink) den += exp2f(load_as_float(sink, h) * 1.4426950408889634f - m_run[a]);   // the sink has no key and no value
    float inv = 1.0f / den;
    const T* grow = gate ? gate + (int64_t)(qstart + i) * ldg : nullptr;
    if (gate_mode == 1) inv *= 1.0f / (1.0f + expf(-load_as_float(grow, h)));
    T* orow = out + (int64_t)(qstart + i) * ldo + (int64_t)h * dv + c0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int c = (b < 4 ? 0 : 64) + 4 * tx + (b & 3);
      if (c < dvc) {
        float val = o[a][b] * inv;
        if (gate_mode == 2) val *= 1.0f / (1.0f + expf(-load_as_float(grow, (int64_t)h * dv + c0 + c)));
        store_from_float(orow, c, val);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------------------------------
constexpr int kLdThreads = 128, kLdTile = 32, kLdMaxRPT = 8;   // latent size <= 128 * 8

// grid (n_head, batch): q'_h = (W_uk[h]^T q_h) * scale * log2(e), r numbers in fp32 -- the query in latent space.
// A thread owns two neighbouring columns of W_uk[h] (dk x r) and one of `groups` slices of its dk rows; the slices are
// summed through shared memory in a fixed order.
constexpr int kAbThreads = 512, kAbMaxChunks = 4;

__host__ __device__ inline int absorb_chunks(int r) { return max(1, min(kAbMaxChunks, (r + 1) / 2 / 32)); }

// grid (n_head, batch, absorb_chunks(r)): every CTA takes a range of column pairs
template <typename T>
__global__ void __launch_bounds__(kAbThreads) latent_absorb_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ w_uk,
                                                                    float* __restrict__ qlat, int dk, int r, float scale_log2, int dk2) {
  // a query head is [dk | dk2]: the first part is absorbed into latent space, the second meets the shared key part stored
  // behind the latent in every cache row, so q' = [W_uk^T q_a | q_b] has r + dk2 numbers
  extern __shared__ __align__(16) float ab_smem[];   // [dk] query, then [groups][2 * ncol] partial sums
  griddep_launch();
  griddep_wait();
  const int h = blockIdx.x, b = blockIdx.y, n_head = gridDim.x, tid = threadIdx.x;
  const int all_pairs = (r + 1) / 2;
  const int ncol = (all_pairs + (int)gridDim.z - 1) / (int)gridDim.z;     // column pairs of this CTA
  const int pair0 = (int)blockIdx.z * ncol;
  const int groups = ncol >= kAbThreads ? 1 : min(kAbThreads / ncol, dk);
  float* const part = ab_smem + dk;
  const T* qh = q + (int64_t)b * ldq + (int64_t)h * (dk + dk2);
  const int R = r + dk2;
  for (int d = tid; d < dk; d += kAbThreads) ab_smem[d] = load_as_float(qh, d);
  if (blockIdx.z == 0)
    for (int d = tid; d < dk2; d += kAbThreads) qlat[((int64_t)b * n_head + h) * R + r + d] = load_as_float(qh, dk + d) * scale_log2;
  __syncthreads();
  const T* w = w_uk + (int64_t)h * dk * r;
  const int per = (dk + groups - 1) / groups;
  for (int item = tid; item < groups * ncol; item += kAbThreads) {
    const int grp = item / ncol, lc = item - grp * ncol, c0 = 2 * (pair0 + lc);
    const bool one = c0 < r, two = c0 + 1 < r;
    const int d1 = min(dk, (grp + 1) * per);
    float a0 = 0.f, a1 = 0.f;
    if (one) {
#pragma unroll 8
      for (int d = grp * per; d < d1; ++d) {
        const float qd = ab_smem[d];
        a0 = fmaf(qd, load_as_float(w, (int64_t)d * r + c0), a0);
        if (two) a1 = fmaf(qd, load_as_float(w, (int64_t)d * r + c0 + 1), a1);
      }
    }
    part[grp * 2 * ncol + 2 * lc] = a0;
    part[grp * 2 * ncol + 2 * lc + 1] = a1;
  }
  __syncthreads();
  for (int lc = tid; lc < 2 * ncol; lc += kAbThreads) {
    const int rr = 2 * pair0 + lc;
    if (rr >= r) continue;
    float acc = 0.f;
    for (int g = 0; g < groups; ++g) acc += part[g * 2 * ncol + lc];
    qlat[((int64_t)b * n_head + h) * R + rr] = acc * scale_log2;
  }
}

// grid (n_split, n_head, batch).  Partial result of one split: r unnormalised latent sums, then the running maximum
// (log2 domain) and the probability sum.
template <typename T>
__global__ void __launch_bounds__(kLdThreads) latent_decode_split_kernel(const float* __restrict__ qlat, const T* __restrict__ cache,
                                                                          int64_t slot_stride, const int* __restrict__ row_slot,
                                                                          const int* __restrict__ row_pos, float* __restrict__ ws, int n_head,
                                                                          int r, int max_seq, int R) {
  // R >= r: numbers per cache row and per q' (the latent, then a key part that enters the scores only)
  extern __shared__ __align__(16) unsigned char ld_smem_raw[];
  griddep_launch();
  griddep_wait();
  float* const ql = reinterpret_cast<float*>(ld_smem_raw);    // [R]  q'
  float* const sc = ql + R;                                    // [32] scores, then probabilities
  float* const st = sc + kLdTile;                              // [4]  running max, sum, rescale factor
  T* const cs = reinterpret_cast<T*>(st + 4);                  // [32][R]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, n_split = gridDim.x, h = blockIdx.y, b = blockIdx.z;
  int ctx = row_pos[b] + 1;
  ctx = ctx < 1 ? 1 : (ctx > max_seq ? max_seq : ctx);
  int per = (ctx + n_split - 1) / n_split;
  per = (per + kLdTile - 1) / kLdTile * kLdTile;
  const int k0 = split * per, k1 = min(ctx, k0 + per);
  const T* crow = cache + (int64_t)row_slot[b] * slot_stride;

  for (int rr = tid; rr < R; rr += kLdThreads) ql[rr] = qlat[((int64_t)b * n_head + h) * R + rr];
  if (tid == 0) { st[0] = -INFINITY; st[1] = 0.f; st[2] = 1.f; }
  float o[kLdMaxRPT];
#pragma unroll
  for (int i = 0; i < kLdMaxRPT; ++i) o[i] = 0.f;

  for (int j0 = k0; j0 < k1; j0 += kLdTile) {
    __syncthreads();   // previous tile consumed; ql visible on the first pass
    const int nj = min(kLdTile, k1 - j0);
    for (int idx = tid; idx < nj * R; idx += kLdThreads) cs[idx] = crow[(int64_t)j0 * R + idx];
    __syncthreads();
    for (int j = warp; j < kLdTile; j += kLdThreads / 32) {
      float dot = 0.f;
      if (j < nj)
        for (int rr = lane; rr < R; rr += 32) dot = fmaf(ql[rr], load_as_float(cs, (int64_t)j * R + rr), dot);
      dot = warp_sum(dot);
      if (lane == 0) sc[j] = j < nj ? dot : -INFINITY;
    }
    __syncthreads();
    if (warp == 0) {
      const float sv = sc[lane];
      const float m_old = st[0];
      const float m_new = fmaxf(m_old, warp_max(sv));   // finite: every tile holds at least one key
      const float p = exp2f(sv - m_new);
      const float psum = warp_sum(p);
      __syncwarp();
      sc[lane] = p;
      if (lane == 0) {
        const float a = exp2f(m_old - m_new);
        st[2] = a;
        st[1] = st[1] * a + psum;
        st[0] = m_new;
      }
    }
    __syncthreads();
    const float a = st[2];
#pragma unroll
    for (int i = 0; i < kLdMaxRPT; ++i) {
      const int rr = tid + i * kLdThreads;
      if (rr < r) {
        float acc = o[i] * a;
        for (int j = 0; j < nj; ++j) acc = fmaf(sc[j], load_as_float(cs, (int64_t)j * R + rr), acc);
        o[i] = acc;
      }
    }
  }
  __syncthreads();
  float* dst = ws + (((int64_t)b * n_head + h) * n_split + split) * (r + 2);
#pragma unroll
  for (int i = 0; i < kLdMaxRPT; ++i) {
    const int rr = tid + i * kLdThreads;
    if (rr < r) dst[rr] = o[i];
  }
  if (tid == 0) { dst[r] = st[0]; dst[r + 1] = st[1]; }
}

// The same split on the tensor cores (bf16, r and R multiples of 32, r <= 512): one CTA takes 16 heads of one sequence, so the
// scores of a 32-key tile are one (16 x r) . (r x 32) product and the probability-weighted latent sum a (16 x 32) . (32 x r)
// product, both mma.sync.m16n8k16 with fp32 accumulation; q' and the probabilities are rounded to bf16 as operands.
// Warp w computes the scores of keys 8 w .. 8 w + 7 and owns columns [w r / 4, (w + 1) r / 4) of the latent sum.
// grid (n_split, ceil(n_head / 16), batch); partial results in the layout of the kernel above.
constexpr int kLmHeads = 16, kLmMaxNT = 16;

__global__ void __launch_bounds__(kLdThreads) latent_decode_mma_kernel(const float* __restrict__ qlat, const __nv_bfloat16* __restrict__ cache,
                                                                        int64_t slot_stride, const int* __restrict__ row_slot,
                                                                        const int* __restrict__ row_pos, float* __restrict__ ws, int n_head,
                                                                        int r, int max_seq, int R) {
  extern __shared__ __align__(16) unsigned char lm_smem_raw[];
  griddep_launch();
  griddep_wait();
  const int pitch = R + 8;                                              // bf16 elements; rows stay 16-byte aligned and spread over the banks
  __nv_bfloat16* const Qs = reinterpret_cast<__nv_bfloat16*>(lm_smem_raw);   // [16][pitch]
  __nv_bfloat16* const Cbuf = Qs + kLmHeads * pitch;                          // [2][32][pitch]: the tile in use and the next one
  __nv_bfloat16* const Ps = Cbuf + 2 * kLdTile * pitch;                       // [16][40]
  float* const smax = reinterpret_cast<float*>(Ps + kLmHeads * 40);          // [4][16]
  float* const ssum = smax + 4 * kLmHeads;                                    // [4][16]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int split = blockIdx.x, n_split = gridDim.x, h0 = blockIdx.y * kLmHeads, b = blockIdx.z;
  int ctx = row_pos[b] + 1;
  ctx = ctx < 1 ? 1 : (ctx > max_seq ? max_seq : ctx);
  int per = (ctx + n_split - 1) / n_split;
  per = (per + kLdTile - 1) / kLdTile * kLdTile;
  const int k0 = split * per, k1 = min(ctx, k0 + per);
  const __nv_bfloat16* crow = cache + (int64_t)row_slot[b] * slot_stride;
  const int nt = r / 32;                                                 // 8-column tiles of the latent sum per warp
  const int chunks = R / 8;                                              // 16-byte chunks per cache row

  auto load_tile = [&](int j0, int buf) {
    const int nj = min(kLdTile, k1 - j0);
    __nv_bfloat16* dst = Cbuf + buf * kLdTile * pitch;
    for (int idx = tid; idx < kLdTile * chunks; idx += kLdThreads) {
      const int j = idx / chunks, c = idx - j * chunks;
      pf_cp16(pf_smem(dst + j * pitch + c * 8), crow + (int64_t)(j0 + (j < nj ? j : 0)) * R + c * 8, j < nj);
    }
    pf_commit();
  };
  if (k0 < k1) load_tile(k0, 0);
  for (int idx = tid; idx < kLmHeads * (R / 4); idx += kLdThreads) {     // q' of the sixteen heads, four values at a time
    const int hh = idx / (R / 4), c4 = idx - hh * (R / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (h0 + hh < n_head) v = *reinterpret_cast<const float4*>(qlat + ((int64_t)b * n_head + h0 + hh) * R + 4 * c4);
    *reinterpret_cast<uint2*>(Qs + hh * pitch + 4 * c4) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  }
  float o[kLmMaxNT][4];
#pragma unroll
  for (int i = 0; i < kLmMaxNT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;             // rows g and g + 8, identical in every warp

  int buf = 0;
  for (int j0 = k0; j0 < k1; j0 += kLdTile, buf ^= 1) {
    __syncthreads();                                                     // the other buffer is free again; Qs visible on the first pass
    const int nj = min(kLdTile, k1 - j0);
    if (j0 + kLdTile < k1) { load_tile(j0 + kLdTile, buf ^ 1); pf_wait<1>(); } else { pf_wait<0>(); }
    __syncthreads();
    const __nv_bfloat16* Cs = Cbuf + buf * kLdTile * pitch;
    // scores of this warp's eight keys for the sixteen heads
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ks = 0; ks < R / 32; ++ks) {
      uint32_t a0[4], a1[4], kb[4];
      ldsm_x4(a0, pf_smem(Qs + (lane & 15) * pitch + ks * 32 + (lane >> 4) * 8));
      ldsm_x4(a1, pf_smem(Qs + (lane & 15) * pitch + ks * 32 + 16 + (lane >> 4) * 8));
      ldsm_x4(kb, pf_smem(Cs + (warp * 8 + (lane & 7)) * pitch + ks * 32 + (lane >> 3) * 8));
      pf_mma(sacc, a0, kb[0], kb[1]);
      pf_mma(sacc, a1, kb[2], kb[3]);
    }
    const int key = warp * 8 + 2 * tq;
    if (key >= nj) sacc[0] = sacc[2] = -INFINITY;
    if (key + 1 >= nj) sacc[1] = sacc[3] = -INFINITY;
    float tA = fmaxf(sacc[0], sacc[1]), tB = fmaxf(sacc[2], sacc[3]);
    tA = fmaxf(tA, __shfl_xor_sync(0xffffffffu, tA, 1)); tA = fmaxf(tA, __shfl_xor_sync(0xffffffffu, tA, 2));
    tB = fmaxf(tB, __shfl_xor_sync(0xffffffffu, tB, 1)); tB = fmaxf(tB, __shfl_xor_sync(0xffffffffu, tB, 2));
    if (tq == 0) { smax[warp * kLmHeads + g] = tA; smax[warp * kLmHeads + g + 8] = tB; }
    __syncthreads();
    float nA = mA, nB = mB;
#pragma unroll
    for (int w = 0; w < 4; ++w) { nA = fmaxf(nA, smax[w * kLmHeads + g]); nB = fmaxf(nB, smax[w * kLmHeads + g + 8]); }
    const float cA = exp2f(mA - nA), cB = exp2f(mB - nB);                // the first key of a split is always visible: nA, nB finite
    const float p0 = exp2f(sacc[0] - nA), p1 = exp2f(sacc[1] - nA), p2 = exp2f(sacc[2] - nB), p3 = exp2f(sacc[3] - nB);
    *reinterpret_cast<uint32_t*>(Ps + g * 40 + key) = pack_bf16(p0, p1);
    *reinterpret_cast<uint32_t*>(Ps + (g + 8) * 40 + key) = pack_bf16(p2, p3);
    float rA = p0 + p1, rB = p2 + p3;
    rA += __shfl_xor_sync(0xffffffffu, rA, 1); rA += __shfl_xor_sync(0xffffffffu, rA, 2);
    rB += __shfl_xor_sync(0xffffffffu, rB, 1); rB += __shfl_xor_sync(0xffffffffu, rB, 2);
    if (tq == 0) { ssum[warp * kLmHeads + g] = rA; ssum[warp * kLmHeads + g + 8] = rB; }
    __syncthreads();
    float sA = 0.f, sB = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { sA += ssum[w * kLmHeads + g]; sB += ssum[w * kLmHeads + g + 8]; }
    lA = lA * cA + sA; lB = lB * cB + sB;
    mA = nA; mB = nB;
    // latent sum: this warp's columns, all 32 keys
    uint32_t pa0[4], pa1[4];
    ldsm_x4(pa0, pf_smem(Ps + (lane & 15) * 40 + (lane >> 4) * 8));
    ldsm_x4(pa1, pf_smem(Ps + (lane & 15) * 40 + 16 + (lane >> 4) * 8));
    const int col0 = warp * (r / 4);
#pragma unroll
    for (int i = 0; i < kLmMaxNT; i += 2) {
      if (i < nt) {
        o[i][0] *= cA; o[i][1] *= cA; o[i][2] *= cB; o[i][3] *= cB;
        o[i + 1][0] *= cA; o[i + 1][1] *= cA; o[i + 1][2] *= cB; o[i + 1][3] *= cB;
        uint32_t v0[4], v1[4];
        const int krow = (((lane >> 3) & 1) << 3) + (lane & 7), col = col0 + i * 8 + (lane >> 4) * 8;
        ldsm_x4_t(v0, pf_smem(Cs + krow * pitch + col));
        ldsm_x4_t(v1, pf_smem(Cs + (16 + krow) * pitch + col));
        pf_mma(o[i], pa0, v0[0], v0[1]);
        pf_mma(o[i + 1], pa0, v0[2], v0[3]);
        pf_mma(o[i], pa1, v1[0], v1[1]);
        pf_mma(o[i + 1], pa1, v1[2], v1[3]);
      }
    }
  }
  const int col0 = warp * (r / 4);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int h = h0 + g + 8 * half;
    if (h >= n_head) continue;
    float* dst = ws + (((int64_t)b * n_head + h) * n_split + split) * (r + 2);
#pragma unroll
    for (int i = 0; i < kLmMaxNT; ++i)
      if (i < nt) {
        dst[col0 + i * 8 + 2 * tq] = o[i][2 * half];
        dst[col0 + i * 8 + 2 * tq + 1] = o[i][2 * half + 1];
      }
    if (warp == 0 && tq == 0) { dst[r] = half ? mB : mA; dst[r + 1] = half ? lB : lA; }
  }
}

// grid (n_head, batch, chunks of the value rows): merge the splits, then out_h = W_uv[h] (sum_j p_j c_j)
constexpr int kLmThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kLmThreads) latent_decode_merge_kernel(const float* __restrict__ ws, const T* __restrict__ w_uv,
                                                                          T* __restrict__ out, int64_t ldo, int n_head, int dv, int r,
                                                                          int n_split, const T* __restrict__ sink, const T* __restrict__ gate,
                                                                          int64_t ldg, int gate_mode) {
  extern __shared__ __align__(16) float lm_smem[];   // [r] averaged latent, [n_split] weights, maxima, sums
  griddep_launch();
  griddep_wait();
  float* const avg = lm_smem;
  float* const wgt = avg + ((r + 3) & ~3);
  float* const smx = wgt + n_split;
  float* const ssm = smx + n_split;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y;
  const float* src = ws + ((int64_t)b * n_head + h) * n_split * (r + 2);
  for (int s = tid; s < n_split; s += kLmThreads) {
    smx[s] = src[(int64_t)s * (r + 2) + r];
    ssm[s] = src[(int64_t)s * (r + 2) + r + 1];
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, smx[s]);
  for (int s = tid; s < n_split; s += kLmThreads) wgt[s] = smx[s] == -INFINITY ? 0.f : exp2f(smx[s] - mx);
  __syncthreads();
  float tot = sink ? exp2f(load_as_float(sink, h) * 1.4426950408889634f - mx) : 0.f;   // a sink joins the denominator only
  for (int s = 0; s < n_split; ++s) tot = fmaf(wgt[s], ssm[s], tot);
  const float inv = 1.0f / tot;
  const T* grow = gate_mode ? gate + (int64_t)b * ldg : nullptr;
  const float head_gate = gate_mode == 1 ? 1.0f / (1.0f + expf(-load_as_float(grow, h))) : 1.0f;
  for (int rr = tid; rr < r; rr += kLmThreads) {
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_split; ++s) acc = fmaf(wgt[s], src[(int64_t)s * (r + 2) + rr], acc);
    avg[rr] = acc * inv;
  }
  __syncthreads();
  // this CTA's share of the head's value rows (gridDim.z CTAs per head)
  const int per = (dv + (int)gridDim.z - 1) / (int)gridDim.z;
  const int c_lo = (int)blockIdx.z * per, c_hi = min(dv, c_lo + per);
#pragma unroll 2
  for (int c = c_lo + warp; c < c_hi; c += kLmThreads / 32) {
    float dot = warp_dot(w_uv + ((int64_t)h * dv + c) * r, avg, r, lane) * head_gate;
    if (lane == 0) {
      if (gate_mode == 2) dot *= 1.0f / (1.0f + expf(-load_as_float(grow, (int64_t)h * dv + c)));
      store_from_float(out, (int64_t)b * ldo + (int64_t)h * dv + c, dot);
    }
  }
}

template <typename T>
int prefill_launch(const b200_latent_prefill_args* a, cudaStream_t st) {
  const int dkp = conflict_free_pitch(a->dk);
  const size_t smem = (size_t)(2 * kLpBM * dkp + kLpBN * kLpDV + kLpBM * (kLpBN + 4)) * sizeof(float);
  B200_CHECK_ARG(smem <= 227 * 1024, "b200_latent_prefill: query-key size %d needs %zu bytes of shared memory", a->dk, smem);
  static PerDeviceOnce once;
  if (once.need()) {
    B200_CUDA(cudaFuncSetAttribute(latent_prefill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    once.done();
  }
  const int nchunk = (a->dv + kLpDV - 1) / kLpDV;
  const dim3 grid((unsigned)((a->max_q_len + kLpBM - 1) / kLpBM), (unsigned)(a->n_head * nchunk), (unsigned)a->n_seqs);
  B200_CUDA(launch(latent_prefill_kernel<T>, grid, dim3(kLpThreads), smem, st, (const T*)a->q, a->ldq, (const T*)a->k, a->ldk, (const T*)a->v,
                   a->ldv, (const int4*)a->seqs, (T*)a->out, a->ldo, a->n_head, a->dk, a->dv, a->scale * 1.4426950408889634f, (const T*)a->k2, a->ldk2,
                   a->k2 ? a->dk2 : 0, (const T*)a->sink, (const T*)(a->gate_mode ? a->gate : nullptr), a->ldg, a->gate ? a->gate_mode : 0));
  return B200_OK;
}

std::atomic<int> g_decode_simt{0};   // test knob: keep bf16 decode on the any-size kernel

template <typename T>
int decode_launch(const b200_latent_decode_args* a, cudaStream_t st) {
  const int ab_chunks = absorb_chunks(a->r);
  const int ab_ncol = ((a->r + 1) / 2 + ab_chunks - 1) / ab_chunks;
  const int ab_groups = ab_ncol >= kAbThreads ? 1 : std::min(kAbThreads / ab_ncol, a->dk);
  const int dk2 = a->dk2 > 0 ? a->dk2 : 0, R = a->r + dk2;   // numbers per cache row and per q'
  const size_t smem0 = ((size_t)a->dk + (size_t)ab_groups * 2 * ab_ncol) * sizeof(float);
  const size_t smem1 = (size_t)(R + kLdTile + 4) * sizeof(float) + (size_t)kLdTile * R * sizeof(T);
  const size_t smem2 = (size_t)(a->r + 4 + 3 * a->n_split) * sizeof(float);
  const int merge_chunks = std::max(1, std::min(4, a->dv / 32));
  const size_t smem3 = (size_t)((kLmHeads + 2 * kLdTile) * (R + 8) + kLmHeads * 40) * 2 + 8 * kLmHeads * sizeof(float);
  B200_CHECK_ARG(smem0 <= 48 * 1024 && smem1 <= 227 * 1024 && smem2 <= 227 * 1024, "b200_latent_decode: sizes need too much shared memory");
  static PerDeviceOnce once;
  if (once.need()) {
    B200_CUDA(cudaFuncSetAttribute(latent_decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    B200_CUDA(cudaFuncSetAttribute(latent_decode_merge_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    B200_CUDA(cudaFuncSetAttribute(latent_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    once.done();
  }
  float* qlat = (float*)a->workspace;
  float* parts = qlat + (size_t)a->batch * a->n_head * R;
  const float scale_log2 = a->scale * 1.4426950408889634f;
  B200_CUDA(launch(latent_absorb_kernel<T>, dim3((unsigned)a->n_head, (unsigned)a->batch, (unsigned)ab_chunks), dim3(kAbThreads), smem0, st, (const T*)a->q, a->ldq,
                   (const T*)a->w_uk, qlat, a->dk, a->r, scale_log2, dk2));
  const bool tensor = std::is_same<T, __nv_bfloat16>::value && a->r % 32 == 0 && R % 32 == 0 && a->r <= 32 * kLmMaxNT && !g_decode_simt.load() &&
                      smem3 <= 227 * 1024 &&
                      (reinterpret_cast<uintptr_t>(a->cache) & 15) == 0 && (a->slot_stride & 7) == 0;
  if (tensor)
    B200_CUDA(launch(latent_decode_mma_kernel, dim3((unsigned)a->n_split, (unsigned)((a->n_head + kLmHeads - 1) / kLmHeads), (unsigned)a->batch),
                     dim3(kLdThreads), smem3, st, (const float*)qlat, (const __nv_bfloat16*)a->cache, a->slot_stride, a->row_slot, a->row_pos, parts,
                     a->n_head, a->r, a->max_seq, R));
  else
    B200_CUDA(launch(latent_decode_split_kernel<T>, dim3((unsigned)a->n_split, (unsigned)a->n_head, (unsigned)a->batch), dim3(kLdThreads), smem1, st,
                     (const float*)qlat, (const T*)a->cache, a->slot_stride, a->row_slot, a->row_pos, parts, a->n_head, a->r, a->max_seq, R));
  B200_CUDA(launch(latent_decode_merge_kernel<T>, dim3((unsigned)a->n_head, (unsigned)a->batch, (unsigned)merge_chunks), dim3(kLmThreads), smem2, st,
                   (const float*)parts, (const T*)a->w_uv, (T*)a->out, a->ldo, a->n_head, a->dv, a->r, a->n_split, (const T*)a->sink,
                   (const T*)(a->gate_mode ? a->gate : nullptr), a->ldg, a->gate ? a->gate_mode : 0));
  return B200_OK;
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_latent_prefill(const b200_latent_prefill_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->q && a->k && a->v && a->seqs && a->out, "b200_latent_prefill: null pointer");
  B200_CHECK_ARG(a->n_seqs > 0 && a->n_seqs <= 65535 && a->max_q_len > 0 && a->n_head > 0 && a->dk > 0 && a->dv > 0,
                 "b200_latent_prefill: bad shape");
  B200_CHECK_ARG((int64_t)a->n_head * ((a->dv + kLpDV - 1) / kLpDV) <= 65535, "b200_latent_prefill: too many heads");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(a->seqs) & 15) == 0, "b200_latent_prefill: the sequence table must start on a 16-byte boundary");
  B200_CHECK_ARG(!a->k2 || (a->dk2 > 0 && a->dk2 < a->dk), "b200_latent_prefill: the shared key part must be shorter than the query head");
  B200_CHECK_ARG(a->gate_mode >= 0 && a->gate_mode <= 2, "b200_latent_prefill: gate mode 0 (none), 1 (per head) or 2 (per output number)");
  if (a->dtype == B200_BF16) return prefill_launch<__nv_bfloat16>(a, (cudaStream_t)stream);
  if (a->dtype == B200_F32) return prefill_launch<float>(a, (cudaStream_t)stream);
  set_error("b200_latent_prefill: dtype must be bf16 or fp32");
  return B200_ERR_INVALID;
}

size_t b200_latent_decode_workspace_bytes(int batch, int n_head, int r, int n_split) {
  return ((size_t)batch * n_head * r + (size_t)batch * n_head * n_split * (r + 2)) * sizeof(float);
}


int b200_latent_decode_tune(int force_any_size_kernel) { return b200::g_decode_simt.exchange(force_any_size_kernel ? 1 : 0); }

int b200_latent_decode(const b200_latent_decode_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->q && a->w_uk && a->w_uv && a->cache && a->row_slot && a->row_pos && a->out && a->workspace,
                 "b200_latent_decode: null pointer");
  B200_CHECK_ARG(a->batch > 0 && a->batch <= 65535 && a->n_head > 0 && a->n_head <= 65535 && a->dk > 0 && a->dv > 0 && a->r > 0 && a->n_split > 0,
                 "b200_latent_decode: bad shape");
  B200_CHECK_ARG(a->r <= kLdThreads * kLdMaxRPT, "b200_latent_decode: latent size %d above %d", a->r, kLdThreads * kLdMaxRPT);
  B200_CHECK_ARG(a->dk2 >= 0 && a->gate_mode >= 0 && a->gate_mode <= 2, "b200_latent_decode: bad shared key part or gate mode");
  B200_CHECK_ARG(a->workspace_bytes >= b200_latent_decode_workspace_bytes(a->batch, a->n_head, a->r + a->dk2, a->n_split),
                 "b200_latent_decode: workspace too small");
  if (a->dtype == B200_BF16) return decode_launch<__nv_bfloat16>(a, (cudaStream_t)stream);
  if (a->dtype == B200_F32) return decode_launch<float>(a, (cudaStream_t)stream);
  set_error("b200_latent_decode: dtype must be bf16 or fp32");
  return B200_ERR_INVALID;
}

}  // extern "C"
