// Causal attention whose scores are MIXED OVER THE HEADS before the softmax ("talking heads"), over cached keys and values:
//
//   s_g(i, j)  = scale * q_g(i) . k_{kv(g)}(j)              raw score of query head g (kv(g) = g / (H / G): grouped heads)
//   s'_h(i, j) = sum_g talk[h, g] * s_g(i, j)               what head h's softmax sees
//   p_h(i, j)  = exp(s'_h) / (exp(sink_h) + sum_{j' <= i} exp(s'_h(i, j')))     the sink has no key and no value
//   o_h(i)     = sum_j p_h(i, j) v_{kv(h)}(j)
//
// The mixing couples the heads of one (query, key) pair, so a CTA owns a few query rows for ALL heads: per tile of 32 keys it
// computes the raw scores head group by head group (the group's key tile in shared memory), mixes them in shared memory, runs
// the online softmax of every (head, row), and accumulates the value sums (kept in shared memory: H x rows x dv numbers) group by
// group.  Prompts use 4 rows per CTA; single rows split their keys over several CTAs.  Each CTA leaves unnormalised sums with
// its running maximum and denominator; a second kernel merges the splits and adds the sink.  Operands bf16 or fp32, all
// arithmetic fp32.  Keys and values are read from the cache rows of the sequence's slot, where the step's own rows already are.
#include <algorithm>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int kTaThreads = 256, kTaBN = 32;

// multiple of 4 floats with pitch / 4 odd: rows one lane apart fall into different 16-byte bank groups
__host__ __device__ inline int ta_pitch(int d) {
  int p = (d + 3) & ~3;
  if (((p >> 2) & 1) == 0) p += 4;
  return p;
}

__host__ __device__ inline size_t ta_smem_floats(int H, int bm, int dk, int dv) {
  const int dkp = ta_pitch(dk), dvp = (dv + 3) & ~3;
  return (size_t)H * bm * dkp + (size_t)kTaBN * (dkp > dvp ? dkp : dvp) + 2 * (size_t)H * bm * kTaBN + (size_t)H * H + 3 * (size_t)H * bm +
         (size_t)H * bm * dv + 8;
}

// four consecutive elements as floats (8- or 16-byte access; the caller has checked the alignment)
__device__ __forceinline__ float4 ta_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ta_load4(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y));
}

// rows j0 .. j0 + 31 of a cache (row stride ld, `width` numbers from column col0) -> tile[32][pitch] as floats; rows from k_hi on and
// the padding columns are zero.  A warp takes every eighth row, its lanes the columns (four at a time when `vec`).
template <typename T>
__device__ __forceinline__ void ta_load_tile(float* tile, const T* base, int64_t ld, int col0, int width, int pitch, int j0, int k_hi, bool vec) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = warp; j < kTaBN; j += kTaThreads / 32) {
    float* dst = tile + j * pitch;
    const bool ok = j0 + j < k_hi;
    const T* src = base + (int64_t)(ok ? j0 + j : 0) * ld + col0;
    if (vec) {
      for (int d = lane * 4; d < pitch; d += 128)
        *reinterpret_cast<float4*>(dst + d) = ok && d < width ? ta_load4(src + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int d = lane; d < pitch; d += 32) dst[d] = ok && d < width ? load_as_float(src, d) : 0.f;
    }
  }
}

// grid (query tiles, splits, sequences)
template <typename T, int BM>
__global__ void __launch_bounds__(kTaThreads) talk_attn_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ kc, int64_t ldk,
                                                                const T* __restrict__ vc, int64_t ldv, const T* __restrict__ talk,
                                                                const int4* __restrict__ seqs, float* __restrict__ ws, int H, int G, int dk,
                                                                int dv, int max_seq, float scale_log2) {
  extern __shared__ __align__(16) float ta_smem[];
  griddep_launch();
  griddep_wait();
  const int4 sq = seqs[blockIdx.z];
  const int qstart = sq.x, qlen = sq.y, pos0 = sq.z, slot = sq.w;
  const int r0 = (int)blockIdx.x * BM;
  if (r0 >= qlen) return;
  const int n_split = gridDim.y, split = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dkp = ta_pitch(dk), dvp = (dv + 3) & ~3, per_g = H / G;
  constexpr int TS = BM * kTaBN;                       // scores of one head in a tile
  float* const Qs = ta_smem;                           // [H][BM][dkp], times scale * log2(e)
  float* const KV = Qs + (size_t)H * BM * dkp;         // [32][dkp] keys, then [32][dvp] values of one head group
  float* const S = KV + (size_t)kTaBN * (dkp > dvp ? dkp : dvp);   // [H][BM][32] raw scores
  float* const P = S + (size_t)H * TS;                 // [H][BM][32] mixed scores, then probabilities
  float* const Tm = P + (size_t)H * TS;                // [H][H]
  float* const Mx = Tm + (size_t)H * H;                // [H][BM] running maxima (log2 domain)
  float* const Ls = Mx + H * BM;                       // [H][BM] running denominators
  float* const Al = Ls + H * BM;                       // [H][BM] rescale factor of the tile
  float* const O = Al + H * BM + ((4 - ((3 * H * BM + H * H) & 3)) & 3);   // [H][BM][dv], 16-byte aligned

  const int last_row = min(r0 + BM, qlen) - 1;
  const int n_keys = min(pos0 + last_row + 1, max_seq);
  int per = (n_keys + n_split - 1) / n_split;
  per = (per + kTaBN - 1) / kTaBN * kTaBN;
  const int k_lo = split * per, k_hi = min(n_keys, k_lo + per);
  const T* kslot = kc + (int64_t)slot * max_seq * ldk;
  const T* vslot = vc + (int64_t)slot * max_seq * ldv;
  const bool kvec = dk % 4 == 0 && ldk % 4 == 0 && (reinterpret_cast<uintptr_t>(kc) & 15) == 0;
  const bool vvec = dv % 4 == 0 && ldv % 4 == 0 && (reinterpret_cast<uintptr_t>(vc) & 15) == 0;

  for (int idx = tid; idx < H * BM * dkp; idx += kTaThreads) {
    const int hh = idx / (BM * dkp), rem = idx - hh * BM * dkp, i = rem / dkp, d = rem - i * dkp;
    float val = 0.f;
    if (r0 + i < qlen && d < dk) val = load_as_float(q, (int64_t)(qstart + r0 + i) * ldq + (int64_t)hh * dk + d) * scale_log2;
    Qs[idx] = val;
  }
  for (int idx = tid; idx < H * H; idx += kTaThreads) Tm[idx] = talk ? load_as_float(talk, idx) : (idx / H == idx % H ? 1.f : 0.f);
  for (int idx = tid; idx < H * BM; idx += kTaThreads) { Mx[idx] = -INFINITY; Ls[idx] = 0.f; }
  for (int idx = tid; idx < H * BM * dv; idx += kTaThreads) O[idx] = 0.f;

  for (int j0 = k_lo; j0 < k_hi; j0 += kTaBN) {
    // raw scores, one group of heads after the other
    for (int g = 0; g < G; ++g) {
      __syncthreads();                                 // the tile buffer is free (and Q is complete on the first pass)
      ta_load_tile(KV, kslot, ldk, g * dk, dk, dkp, j0, k_hi, kvec);
      __syncthreads();
      const float* krow = KV + lane * dkp;
      for (int pair = warp; pair < per_g * BM; pair += kTaThreads / 32) {   // a warp: one (head, row), its lanes the 32 keys
        const int hq = g * per_g + pair / BM, i = pair % BM;
        const float* qrow = Qs + ((size_t)hq * BM + i) * dkp;
        float acc = 0.f;
        for (int d = 0; d < dkp; d += 4) {
          const float4 a = *reinterpret_cast<const float4*>(qrow + d), b = *reinterpret_cast<const float4*>(krow + d);
          acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
        }
        S[(size_t)hq * TS + i * kTaBN + lane] = acc;
      }
    }
    __syncthreads();
    // mix over the heads, then hide what the row may not see
    for (int e = tid; e < H * TS; e += kTaThreads) {
      const int h = e / TS, rem = e - h * TS, i = rem / kTaBN, key = j0 + (rem & (kTaBN - 1));
      float acc = 0.f;
      for (int g = 0; g < H; ++g) acc = fmaf(Tm[h * H + g], S[(size_t)g * TS + rem], acc);
      const bool seen = key < k_hi && r0 + i < qlen && key <= pos0 + r0 + i;
      P[e] = seen ? acc : -INFINITY;
    }
    __syncthreads();
    for (int row = warp; row < H * BM; row += kTaThreads / 32) {
      const float sv = P[(size_t)row * kTaBN + lane];
      const float m_old = Mx[row];
      const float m_new = fmaxf(m_old, warp_max(sv));
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float p = exp2f(sv - m_safe);
      const float psum = warp_sum(p);
      P[(size_t)row * kTaBN + lane] = p;
      if (lane == 0) {
        const float a = exp2f(m_old - m_safe);         // exp2(-inf) = 0 before the first visible key
        Al[row] = a;
        Ls[row] = Ls[row] * a + psum;
        Mx[row] = m_new;
      }
    }
    // value sums, one group of heads after the other
    for (int g = 0; g < G; ++g) {
      __syncthreads();                                 // the tile buffer is free; probabilities and factors are complete
      ta_load_tile(KV, vslot, ldv, g * dv, dv, dvp, j0, k_hi, vvec);
      __syncthreads();
      if (vvec) {   // four neighbouring value columns per thread: one 16-byte read of V per key serves 4 x BM sums
        for (int item = tid; item < per_g * (dv / 4); item += kTaThreads) {
          const int hq = g * per_g + item / (dv / 4), c = (item % (dv / 4)) * 4;
          float acc[BM][4];
#pragma unroll
          for (int i = 0; i < BM; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
          const float* pr = P + (size_t)hq * TS;
#pragma unroll 4
          for (int j = 0; j < kTaBN; ++j) {
            const float4 v = *reinterpret_cast<const float4*>(KV + j * dvp + c);
#pragma unroll
            for (int i = 0; i < BM; ++i) {
              const float p = pr[i * kTaBN + j];
              acc[i][0] = fmaf(p, v.x, acc[i][0]); acc[i][1] = fmaf(p, v.y, acc[i][1]);
              acc[i][2] = fmaf(p, v.z, acc[i][2]); acc[i][3] = fmaf(p, v.w, acc[i][3]);
            }
          }
#pragma unroll
          for (int i = 0; i < BM; ++i) {
            float* o = O + ((size_t)hq * BM + i) * dv + c;
            const float a = Al[hq * BM + i];
            o[0] = o[0] * a + acc[i][0]; o[1] = o[1] * a + acc[i][1]; o[2] = o[2] * a + acc[i][2]; o[3] = o[3] * a + acc[i][3];
          }
        }
      } else
      for (int item = tid; item < per_g * dv; item += kTaThreads) {
        const int hq = g * per_g + item / dv, c = item % dv;
        float acc[BM];
#pragma unroll
        for (int i = 0; i < BM; ++i) acc[i] = 0.f;
        const float* pr = P + (size_t)hq * TS;
        for (int j = 0; j < kTaBN; ++j) {
          const float v = KV[j * dvp + c];
#pragma unroll
          for (int i = 0; i < BM; ++i) acc[i] = fmaf(pr[i * kTaBN + j], v, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < BM; ++i) {
          float* o = O + ((size_t)hq * BM + i) * dv + c;
          *o = *o * Al[hq * BM + i] + acc[i];
        }
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < H * BM * dv; e += kTaThreads) {
    const int hq = e / (BM * dv), rem = e - hq * BM * dv, i = rem / dv, c = rem - i * dv;
    if (r0 + i < qlen) ws[(((int64_t)(qstart + r0 + i) * H + hq) * n_split + split) * (dv + 2) + c] = O[e];
  }
  for (int e = tid; e < H * BM; e += kTaThreads) {
    const int hq = e / BM, i = e - hq * BM;
    if (r0 + i < qlen) {
      float* dst = ws + (((int64_t)(qstart + r0 + i) * H + hq) * n_split + split) * (dv + 2) + dv;
      dst[0] = Mx[e];
      dst[1] = Ls[e];
    }
  }
}

// one CTA per (row, head): the splits' sums brought to one maximum, the sink joined to the denominator.  The splits' weights are
// worked out once in shared memory; then a thread owns output columns and walks the splits with independent loads.
constexpr int kTmThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kTmThreads) talk_attn_merge_kernel(const float* __restrict__ ws, const T* __restrict__ sink, T* __restrict__ out,
                                                                      int64_t ldo, int H, int dv, int n_split) {
  extern __shared__ __align__(16) float tm_smem[];   // [n_split] weights
  __shared__ float s_red[kTmThreads / 32];
  __shared__ float s_val[2];
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t item = blockIdx.x;
  const int64_t row = item / H;
  const int h = (int)(item - row * H);
  const float* src = ws + item * n_split * (dv + 2);
  const float sink_l = sink ? load_as_float(sink, h) * 1.4426950408889634f : -INFINITY;
  float mx = sink_l;
  for (int s = tid; s < n_split; s += kTmThreads) mx = fmaxf(mx, src[(int64_t)s * (dv + 2) + dv]);
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));      // finite: some split saw a key
  float part = 0.f;
  for (int s = tid; s < n_split; s += kTmThreads) {
    const float m = src[(int64_t)s * (dv + 2) + dv];
    const float w = m == -INFINITY ? 0.f : exp2f(m - mx);
    tm_smem[s] = w;
    part = fmaf(w, src[(int64_t)s * (dv + 2) + dv + 1], part);
  }
  part = warp_sum(part);
  __syncthreads();                                                       // s_red has been read by everyone
  if (lane == 0) s_red[warp] = part;
  __syncthreads();
  if (tid == 0) s_val[0] = 1.0f / (s_red[0] + s_red[1] + s_red[2] + s_red[3] + (sink ? exp2f(sink_l - mx) : 0.f));
  __syncthreads();
  const float inv = s_val[0];
  for (int c = tid; c < dv; c += kTmThreads) {
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < n_split; ++s) acc = fmaf(tm_smem[s], src[(int64_t)s * (dv + 2) + c], acc);
    store_from_float(out, row * ldo + (int64_t)h * dv + c, acc * inv);
  }
}

template <typename T, int BM>
int talk_launch(const b200_talk_attn_args* a, cudaStream_t st, size_t smem) {
  static PerDeviceOnce once;
  if (once.need()) {
    B200_CUDA(cudaFuncSetAttribute(talk_attn_kernel<T, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    once.done();
  }
  const dim3 grid((unsigned)((a->max_q_len + BM - 1) / BM), (unsigned)a->n_split, (unsigned)a->n_seqs);
  B200_CUDA(launch(talk_attn_kernel<T, BM>, grid, dim3(kTaThreads), smem, st, (const T*)a->q, a->ldq, (const T*)a->k_cache, a->ldk, (const T*)a->v_cache,
                   a->ldv, (const T*)a->talk, (const int4*)a->seqs, (float*)a->workspace, a->n_head, a->n_kv_head, a->dk, a->dv, a->max_seq,
                   a->scale * 1.4426950408889634f));
  return B200_OK;
}

template <typename T>
int talk_run(const b200_talk_attn_args* a, cudaStream_t st) {
  // four rows per CTA for prompts when they fit (two resident CTAs preferred), else fewer; single rows always alone
  int bm = 1;
  if (a->max_q_len > 1) {
    for (int cand : {4, 2}) {
      if (ta_smem_floats(a->n_head, cand, a->dk, a->dv) * sizeof(float) <= 227 * 1024) { bm = cand; break; }
    }
  }
  const size_t smem = ta_smem_floats(a->n_head, bm, a->dk, a->dv) * sizeof(float);
  B200_CHECK_ARG(smem <= 227 * 1024, "b200_talk_attn: %d heads of %d / %d numbers need %zu bytes of shared memory", a->n_head, a->dk, a->dv, smem);
  int rc = bm == 4 ? talk_launch<T, 4>(a, st, smem) : bm == 2 ? talk_launch<T, 2>(a, st, smem) : talk_launch<T, 1>(a, st, smem);
  if (rc != B200_OK) return rc;
  const int64_t items = a->rows * a->n_head;
  B200_CUDA(launch(talk_attn_merge_kernel<T>, dim3((unsigned)items), dim3(kTmThreads), (size_t)a->n_split * sizeof(float), st, (const float*)a->workspace,
                   (const T*)a->sink, (T*)a->out, a->ldo, a->n_head, a->dv, a->n_split));
  return B200_OK;
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_talk_attn_workspace_bytes(int64_t rows, int n_head, int dv, int n_split) {
  return (size_t)rows * n_head * n_split * (dv + 2) * sizeof(float);
}

int b200_talk_attn(const b200_talk_attn_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->q && a->k_cache && a->v_cache && a->out && a->seqs && a->workspace, "b200_talk_attn: null pointer");
  B200_CHECK_ARG(a->n_seqs > 0 && a->n_seqs <= 65535 && a->max_q_len > 0 && a->rows > 0 && a->n_head > 0 && a->n_kv_head > 0 &&
                     a->n_head % a->n_kv_head == 0 && a->dk > 0 && a->dv > 0 && a->max_seq > 0 && a->n_split > 0 && a->n_split <= 65535,
                 "b200_talk_attn: bad shape");
  B200_CHECK_ARG(a->rows * a->n_head <= 0x7fffffff, "b200_talk_attn: too many rows");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(a->seqs) & 15) == 0, "b200_talk_attn: the sequence table must start on a 16-byte boundary");
  B200_CHECK_ARG(a->workspace_bytes >= b200_talk_attn_workspace_bytes(a->rows, a->n_head, a->dv, a->n_split), "b200_talk_attn: workspace too small");
  if (a->dtype == B200_BF16) return talk_run<__nv_bfloat16>(a, (cudaStream_t)stream);
  if (a->dtype == B200_F32) return talk_run<float>(a, (cudaStream_t)stream);
  set_error("b200_talk_attn: dtype must be bf16 or fp32");
  return B200_ERR_INVALID;
}

}  // extern "C"
