// Prefill attention over the GQA-native KV cache (T > 1 query tokens), replacing the library SDPA call.
//
// Replaces CausalSelfAttention.scaled_dot_product_attention for the cached multi-token call
// (lit_gpt/model.py:646-665): q (B, H, T, hs) already roped, keys/values read from the caches
// (B, G, Tmax, hs) that b200_rope_kv_append has just extended.  Query row t sees cache positions j <= pos[t]
// -- exactly the rows `mask_cache.index_select(2, input_pos)` selects (model.py:509, 802-804) -- so chunked
// prefill (pos not starting at 0) works; positions past pos[t] are never read.  Softmax in fp32 with a running
// maximum (online softmax), probabilities rounded to bf16 for the P.V product like the fused SDPA back ends.
//
// One CTA = 128 query rows of one head (8 warps x 16 rows), key tiles of 64 positions double-buffered in shared
// memory by cp.async; S = Q K^T and O += P V on mma.sync.m16n8k16 (bf16 -> fp32) with ldmatrix operand loads from
// XOR-swizzled tiles.  The heads of one query group run in adjacent CTAs so the K/V tiles are shared through L2.
// Output is written as (B, T, H * hs), the layout attn.proj consumes (model.py:653).
#include "mma_tile.cuh"

namespace b200 {

namespace {

constexpr int kPfBM = 128;   // query rows per CTA
constexpr int kPfBN = 64;    // keys per tile
constexpr int kPfThreads = 256;

// Where the operands live, in elements.  The cached layout of the GQA models is (B, H or G, rows, HS); a ragged batch packs the
// query rows of all sequences into one (rows, H * HS) matrix and gives, per sequence, seqs[b] = {first query row, query rows,
// position of the first query row, row of position 0 in k / v} -- the positions are then pos0 + row and no pos array is read.
struct PfView {
  int64_t q_b, q_h, q_r;
  int64_t k_b, k_h, k_r;
  int64_t v_b, v_h, v_r;
  int64_t y_b, y_r;
  const int4* seqs;
  // ragged only.  window > 0: row at position i sees keys i - window < j <= i.  sink: one logit per head that joins the softmax
  // denominator (no key, no value, not scaled).  kv_first_row: the sequences start at position 0 and k / v hold exactly the
  // step's rows, so a sequence's keys start at its first query row (seqs[b].w is then free for the caller's own use).
  int window;
  const __nv_bfloat16* sink;
  int kv_first_row;
  // ragged only, kernels instantiated with HK2 > 0: a second key part of HK2 numbers per position shared by all heads (k2, rows k2_r
  // apart, the same rows as k), met by columns [HS, HS + HK2) of each query head.  gate: rows gate_r apart; the output is multiplied
  // by sigmoid(gate[row, h]) (gate_mode 1) or sigmoid(gate[row, h * HS + c]) (gate_mode 2).
  const __nv_bfloat16* k2;
  int64_t k2_r;
  const __nv_bfloat16* gate;
  int64_t gate_r;
  int gate_mode;
  // ragged only, kernels instantiated with MODE 1 or 2: fp32 score planes, one per head (s_h floats apart), already times scale *
  // log2(e).  A plane is a run of 128 x 64 tiles, tile (sequence b, query tile mt, key tile kt) at ((b * s_qt + mt) * s_kt + kt) * 8192,
  // each stored in the accumulator layout of the warp that owns it: [warp][8-key step][lane][4], so a lane's four numbers are one
  // 16-byte access and a warp's access is contiguous.  MODE 1 writes the raw scores of every tile it visits and stops; MODE 2 reads
  // them back (after another kernel has worked on them) instead of multiplying q and k.  kv_slot_rows > 0: seqs[b].w is a cache slot
  // and position 0 of the sequence is row w * kv_slot_rows of k / v.
  float* sbuf;
  int64_t s_h;
  int s_qt, s_kt;
  int64_t kv_slot_rows;
  // ragged only: a distance bias, score -= dist_r1[h] * ln(1 + dist_r2[h] * (i - j)) (both NULL: none).  bias_n > 0: the CTA tabulates
  // the bias of the distances [0, bias_n) in shared memory behind its tiles (bias_n covers every visible distance); 0: computed in place.
  const __nv_bfloat16* dist_r1;
  const __nv_bfloat16* dist_r2;
  int bias_n;
};

constexpr int kPfBiasTabMax = 8192;   // distances a CTA tabulates at most (32 KB)

template <int HS, typename PosT, int HK2 = 0, int MODE = 0>
__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                    const PosT* __restrict__ pos, __nv_bfloat16* __restrict__ y, int T, int n_head, int n_groups, int max_seq,
                    float scale_log2, PfView vw) {
  extern __shared__ __align__(128) uint8_t pf_smem_raw[];
  constexpr int CH = HS / 8;                         // 16-byte chunks per row
  constexpr int QB = kPfBM * HS * 2, KB = kPfBN * HS * 2;
  uint8_t* const sQ = pf_smem_raw;                   // [128][HS]
  uint8_t* const sK = sQ + QB;                       // [2][64][HS]
  uint8_t* const sV = sK + 2 * KB;                   // [2][64][HS]
  constexpr int CH2 = HK2 / 8, KB2 = kPfBN * HK2 * 2;
  uint8_t* const sQ2 = sV + 2 * KB;                  // [128][HK2]  the query columns that meet the shared key part
  uint8_t* const sK2 = sQ2 + kPfBM * HK2 * 2;        // [2][64][HK2]
  float* const sTab = reinterpret_cast<float*>(sK2 + 2 * KB2);   // [bias_n] distance bias by distance, in units of the raw dot product
  __shared__ int s_maxpos[kPfThreads / 32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int mt = (int)gridDim.x - 1 - (int)blockIdx.x;     // long (late) query tiles are scheduled first
  const int h = blockIdx.y, b = blockIdx.z;
  const int grp = h / (n_head / n_groups);
  const int r0 = mt * kPfBM;
  griddep_launch();
  griddep_wait();
  int pos0 = 0;
  int64_t qrow0 = 0, kvrow0 = 0;
  if (vw.seqs) {   // ragged: this sequence's own length, first position and places in the packed operands
    const int4 sq = vw.seqs[b];
    T = sq.y;
    pos0 = sq.z;
    max_seq = sq.z + sq.y;
    qrow0 = sq.x;
    kvrow0 = vw.kv_first_row ? sq.x : (vw.kv_slot_rows > 0 ? (int64_t)sq.w * vw.kv_slot_rows : sq.w);
    if (r0 >= T) return;
  }

  const __nv_bfloat16* qh = q + (int64_t)b * vw.q_b + (int64_t)h * vw.q_h + qrow0 * vw.q_r;
  const __nv_bfloat16* kg = kc + (int64_t)b * vw.k_b + (int64_t)grp * vw.k_h + kvrow0 * vw.k_r;
  const __nv_bfloat16* vg = vc + (int64_t)b * vw.v_b + (int64_t)grp * vw.v_h + kvrow0 * vw.v_r;
  const __nv_bfloat16* k2g = HK2 > 0 ? vw.k2 + kvrow0 * vw.k2_r : nullptr;

  // this thread's two query rows and their causal limits; the CTA's key range is [0, max limit]
  const int rowA = r0 + warp * 16 + g, rowB = rowA + 8;
  auto clampp = [&](int r) -> int {
    if (r >= T) return -1;
    int64_t v = vw.seqs ? (int64_t)pos0 + r : (int64_t)pos[r];
    return (int)(v < 0 ? 0 : (v >= max_seq ? max_seq - 1 : v));
  };
  const int limA = clampp(rowA), limB = clampp(rowB);
  int wl = max(limA, limB);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wl = max(wl, __shfl_xor_sync(0xffffffffu, wl, o));
  if (lane == 0) s_maxpos[warp] = wl;

  // Q tile -> shared (rows past T are zero-filled)
  if constexpr (MODE != 2)
  for (int i = tid; i < kPfBM * CH; i += kPfThreads) {
    const int r = i / CH, c = i % CH;
    const bool ok = r0 + r < T;
    pf_cp16(pf_smem(sQ) + sw<HS>(r, c), qh + (int64_t)(ok ? r0 + r : 0) * vw.q_r + c * 8, ok);
  }
  if constexpr (HK2 > 0) {
    for (int i = tid; i < kPfBM * CH2; i += kPfThreads) {
      const int r = i / CH2, c = i % CH2;
      const bool ok = r0 + r < T;
      pf_cp16(pf_smem(sQ2) + sw<HK2>(r, c), qh + (int64_t)(ok ? r0 + r : 0) * vw.q_r + HS + c * 8, ok);
    }
  }
  pf_commit();
  __syncthreads();
  int cta_lim = -1;
#pragma unroll
  for (int w = 0; w < kPfThreads / 32; ++w) cta_lim = max(cta_lim, s_maxpos[w]);
  const int ntiles = (cta_lim + kPfBN) / kPfBN;      // cta_lim >= 0 because r0 < T
  const int window = vw.seqs ? vw.window : 0;
  // with a window the first rows of the tile decide where the key range starts (ragged positions grow with the row)
  const int tile_lo = window > 0 ? max(0, pos0 + r0 - window + 1) / kPfBN : 0;
  const int loA = window > 0 ? limA - window + 1 : 0, loB = window > 0 ? limB - window + 1 : 0;
  const int warp_lo = window > 0 ? pos0 + r0 + warp * 16 - window + 1 : 0;     // lowest key any row of this warp sees

  auto load_kv = [&](int tile, int buf) {
    const int j0 = tile * kPfBN;
    for (int i = tid; i < kPfBN * CH; i += kPfThreads) {
      const int r = i / CH, c = i % CH;
      const bool ok = j0 + r <= cta_lim;
      const int64_t row = ok ? j0 + r : 0;
      if constexpr (MODE != 2) pf_cp16(pf_smem(sK) + buf * KB + sw<HS>(r, c), kg + row * vw.k_r + c * 8, ok);
      if constexpr (MODE != 1) pf_cp16(pf_smem(sV) + buf * KB + sw<HS>(r, c), vg + row * vw.v_r + c * 8, ok);
    }
    if constexpr (HK2 > 0) {
      for (int i = tid; i < kPfBN * CH2; i += kPfThreads) {
        const int r = i / CH2, c = i % CH2;
        const bool ok = j0 + r <= cta_lim;
        pf_cp16(pf_smem(sK2) + buf * KB2 + sw<HK2>(r, c), k2g + (ok ? j0 + r : 0) * vw.k2_r + c * 8, ok);
      }
    }
    pf_commit();
  };
  load_kv(tile_lo, tile_lo & 1);

  float o_acc[HS / 8][4];
#pragma unroll
  for (int i = 0; i < HS / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

  // distance bias on the raw dot products: (s - r1 log2(1 + r2 dist) / scale_log2) * scale_log2 is the biased score in the log2 domain
  const bool biased = MODE == 0 && vw.seqs && vw.dist_r1;
  const float r1q = biased ? __bfloat162float(vw.dist_r1[h]) / scale_log2 : 0.f, r2h = biased ? __bfloat162float(vw.dist_r2[h]) : 0.f;
  const int ntab = biased ? vw.bias_n : 0;
  for (int i = tid; i < ntab; i += kPfThreads) sTab[i] = r1q * log2f(fmaf(r2h, (float)i, 1.0f));

  // Q fragments stay in registers for the whole key loop
  pf_wait<1>();
  __syncthreads();
  uint32_t qf[MODE == 2 ? 1 : HS / 16][4];
  if constexpr (MODE != 2) {
#pragma unroll
    for (int ks = 0; ks < HS / 16; ++ks)
      ldsm_x4(qf[ks], pf_smem(sQ) + sw<HS>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
  }
  // this lane's place in the first key tile of its query tile's run of the score plane
  float* const plane = MODE != 0 ? vw.sbuf + (int64_t)h * vw.s_h + ((int64_t)b * vw.s_qt + mt) * vw.s_kt * (kPfBM * kPfBN) + (warp * 256 + lane) * 4 : nullptr;
  uint32_t qf2[HK2 > 0 ? HK2 / 16 : 1][4];
  if constexpr (HK2 > 0) {
#pragma unroll
    for (int ks = 0; ks < HK2 / 16; ++ks)
      ldsm_x4(qf2[ks], pf_smem(sQ2) + sw<HK2>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
  }

  const int warp_lim = wl;
  for (int tile = tile_lo; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) { load_kv(tile + 1, buf ^ 1); pf_wait<1>(); } else { pf_wait<0>(); }
    __syncthreads();
    const int j0 = tile * kPfBN;
    if (j0 <= warp_lim && j0 + kPfBN > warp_lo) {   // warp-uniform: tiles entirely above this warp's rows, or below their windows, contribute nothing
      float s[kPfBN / 8][4];
#pragma unroll
      for (int i = 0; i < kPfBN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      const uint32_t kb = pf_smem(sK) + buf * KB, vb = pf_smem(sV) + buf * KB;
      if constexpr (MODE == 2) {   // the scores were computed (and worked on) before: fetch this thread's share of the tile
        const float* tp = plane + (int64_t)tile * (kPfBM * kPfBN);
#pragma unroll
        for (int i = 0; i < kPfBN / 8; ++i) {
          const float4 v = *reinterpret_cast<const float4*>(tp + i * 128);
          s[i][0] = v.x; s[i][1] = v.y; s[i][2] = v.z; s[i][3] = v.w;
        }
      } else {
#pragma unroll
      for (int ks = 0; ks < HS / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < kPfBN / 16; ++np) {
          uint32_t kf[4];
          ldsm_x4(kf, kb + sw<HS>(np * 16 + ((lane >> 4) << 3) + (lane & 7), ks * 2 + ((lane >> 3) & 1)));
          pf_mma(s[2 * np], qf[ks], kf[0], kf[1]);
          pf_mma(s[2 * np + 1], qf[ks], kf[2], kf[3]);
        }
      }
      }
      if constexpr (MODE == 1) {   // leave the raw scores (times scale * log2 e) in the plane; the rest happens in later launches
        float* tp = plane + (int64_t)tile * (kPfBM * kPfBN);
#pragma unroll
        for (int i = 0; i < kPfBN / 8; ++i)
          *reinterpret_cast<float4*>(tp + i * 128) = make_float4(s[i][0] * scale_log2, s[i][1] * scale_log2, s[i][2] * scale_log2, s[i][3] * scale_log2);
      } else {
      if constexpr (HK2 > 0) {   // the shared key part's share of the scores
        const uint32_t kb2 = pf_smem(sK2) + buf * KB2;
#pragma unroll
        for (int ks = 0; ks < HK2 / 16; ++ks) {
#pragma unroll
          for (int np = 0; np < kPfBN / 16; ++np) {
            uint32_t kf[4];
            ldsm_x4(kf, kb2 + sw<HK2>(np * 16 + ((lane >> 4) << 3) + (lane & 7), ks * 2 + ((lane >> 3) & 1)));
            pf_mma(s[2 * np], qf2[ks], kf[0], kf[1]);
            pf_mma(s[2 * np + 1], qf2[ks], kf[2], kf[3]);
          }
        }
      }
      // causal limit + running maximum
      const bool need_mask = j0 + kPfBN - 1 > min(limA < 0 ? 0x7fffffff : limA, limB < 0 ? 0x7fffffff : limB) || limA < 0 || limB < 0 ||
                             (window > 0 && j0 < max(loA, loB));
      float tmA = -INFINITY, tmB = -INFINITY;
      if (biased) {
        // The bias depends on row - key only, and this thread's second row lies 8 below its first: entry (i, c) of the first row is
        // e - 8 (i + 1) - c away from its key, of the second e - 8 i - c, so 18 values serve the thread's 32 entries.  Entries ahead of
        // a row (negative distance) or beyond the table get a neighbour's value and are masked below.
        const int e = limA + 8 - j0 - 2 * tq;
        float vb[kPfBN / 8 + 1][2];
#pragma unroll
        for (int m = 0; m <= kPfBN / 8; ++m) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int dd = max(e - 8 * m - c, 0);
            vb[m][c] = ntab > 0 ? sTab[min(dd, ntab - 1)] : r1q * log2f(fmaf(r2h, (float)dd, 1.0f));
          }
        }
#pragma unroll
        for (int i = 0; i < kPfBN / 8; ++i) {
          s[i][0] -= vb[i + 1][0];
          s[i][1] -= vb[i + 1][1];
          s[i][2] -= vb[i][0];
          s[i][3] -= vb[i][1];
        }
      }
#pragma unroll
      for (int i = 0; i < kPfBN / 8; ++i) {
        if (need_mask) {
          const int j = j0 + i * 8 + 2 * tq;
          if (j > limA || j < loA) s[i][0] = -INFINITY;
          if (j + 1 > limA || j + 1 < loA) s[i][1] = -INFINITY;
          if (j > limB || j < loB) s[i][2] = -INFINITY;
          if (j + 1 > limB || j + 1 < loB) s[i][3] = -INFINITY;
        }
        tmA = fmaxf(tmA, fmaxf(s[i][0], s[i][1]));
        tmB = fmaxf(tmB, fmaxf(s[i][2], s[i][3]));
      }
      tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1)); tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
      tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1)); tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
      const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
      // rows with nothing visible yet keep m = -inf: use 0 as the exponent origin so that exp2(-inf - 0) = 0
      const float oA = nmA == -INFINITY ? 0.f : nmA * scale_log2, oB = nmB == -INFINITY ? 0.f : nmB * scale_log2;
      const float cA = mA == -INFINITY ? 0.f : exp2f(mA * scale_log2 - oA), cB = mB == -INFINITY ? 0.f : exp2f(mB * scale_log2 - oB);
      mA = nmA; mB = nmB;
      float rsA = 0.f, rsB = 0.f;
      uint32_t pfr[kPfBN / 16][4];
#pragma unroll
      for (int i = 0; i < kPfBN / 8; ++i) {
        const float p0 = exp2f(fmaf(s[i][0], scale_log2, -oA)), p1 = exp2f(fmaf(s[i][1], scale_log2, -oA));
        const float p2 = exp2f(fmaf(s[i][2], scale_log2, -oB)), p3 = exp2f(fmaf(s[i][3], scale_log2, -oB));
        rsA += p0 + p1; rsB += p2 + p3;
        pfr[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
        pfr[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      lA = lA * cA + rsA; lB = lB * cB + rsB;
#pragma unroll
      for (int i = 0; i < HS / 8; ++i) { o_acc[i][0] *= cA; o_acc[i][1] *= cA; o_acc[i][2] *= cB; o_acc[i][3] *= cB; }
#pragma unroll
      for (int ks = 0; ks < kPfBN / 16; ++ks) {
#pragma unroll
        for (int dp = 0; dp < HS / 16; ++dp) {
          uint32_t vf[4];
          ldsm_x4_t(vf, vb + sw<HS>(ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7), dp * 2 + (lane >> 4)));
          pf_mma(o_acc[2 * dp], pfr[ks], vf[0], vf[1]);
          pf_mma(o_acc[2 * dp + 1], pfr[ks], vf[2], vf[3]);
        }
      }
      }   // MODE != 1
    }
    __syncthreads();   // the buffer just read is refilled by the next iteration's prefetch
  }

  if constexpr (MODE == 1) return;
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  float iA = lA > 0.f ? 1.f / lA : 0.f, iB = lB > 0.f ? 1.f / lB : 0.f;
  if (vw.seqs && vw.sink) {   // the sink joins the denominator once: l is in units of exp2(m * scale_log2)
    const float sk = __bfloat162float(vw.sink[h]) * 1.4426950408889634f;
    const float eA = mA == -INFINITY ? sk : fmaxf(mA * scale_log2, sk), eB = mB == -INFINITY ? sk : fmaxf(mB * scale_log2, sk);
    const float cA = mA == -INFINITY ? 0.f : exp2f(mA * scale_log2 - eA), cB = mB == -INFINITY ? 0.f : exp2f(mB * scale_log2 - eB);
    iA = cA / (lA * cA + exp2f(sk - eA));
    iB = cB / (lB * cB + exp2f(sk - eB));
  }
  const int gmode = vw.seqs && vw.gate ? vw.gate_mode : 0;
  // the gate's sigmoid with the fast exponential and reciprocal: the product is rounded to bf16 right after
  auto sigf = [](float z) -> float { return __fdividef(1.0f, 1.0f + __expf(-z)); };
  auto sigm = [&](const __nv_bfloat16* p) -> float { return sigf(__bfloat162float(*p)); };
  // a pair of neighbouring gates as one 4-byte load when every pair starts on a 4-byte boundary
  const bool gate_pairs = gmode == 2 && (reinterpret_cast<uintptr_t>(vw.gate) & 3) == 0 && (vw.gate_r & 1) == 0;
  auto gate2 = [&](const __nv_bfloat16* p, float& a0, float& a1) {
    if (gate_pairs) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
      a0 *= sigf(bf16lo(v));
      a1 *= sigf(bf16hi(v));
    } else {
      a0 *= sigm(p);
      a1 *= sigm(p + 1);
    }
  };
  if (rowA < T) {
    __nv_bfloat16* yr = y + (int64_t)b * vw.y_b + (qrow0 + rowA) * vw.y_r + (int64_t)h * HS;
    const __nv_bfloat16* gr = gmode ? vw.gate + (qrow0 + rowA) * vw.gate_r : nullptr;
    if (gmode == 1) iA *= sigm(gr + h);
#pragma unroll
    for (int i = 0; i < HS / 8; ++i) {
      float a0 = o_acc[i][0] * iA, a1 = o_acc[i][1] * iA;
      if (gmode == 2) gate2(gr + (int64_t)h * HS + i * 8 + 2 * tq, a0, a1);
      *reinterpret_cast<uint32_t*>(yr + i * 8 + 2 * tq) = pack_bf16(a0, a1);
    }
  }
  if (rowB < T) {
    __nv_bfloat16* yr = y + (int64_t)b * vw.y_b + (qrow0 + rowB) * vw.y_r + (int64_t)h * HS;
    const __nv_bfloat16* gr = gmode ? vw.gate + (qrow0 + rowB) * vw.gate_r : nullptr;
    if (gmode == 1) iB *= sigm(gr + h);
#pragma unroll
    for (int i = 0; i < HS / 8; ++i) {
      float a0 = o_acc[i][2] * iB, a1 = o_acc[i][3] * iB;
      if (gmode == 2) gate2(gr + (int64_t)h * HS + i * 8 + 2 * tq, a0, a1);
      *reinterpret_cast<uint32_t*>(yr + i * 8 + 2 * tq) = pack_bf16(a0, a1);
    }
  }
}

template <int HS, typename PosT, int HK2 = 0, int MODE = 0>
cudaError_t launch_prefill(const void* q, const void* kc, const void* vc, const void* pos, void* y, int B, int T, int H, int G, int max_seq,
                           float scale, cudaStream_t st, const PfView* view = nullptr) {
  // default: q (B, H, T, HS), caches (B, G, max_seq, HS), y (B, T, H * HS)
  const PfView vw = view ? *view
                         : PfView{(int64_t)H * T * HS, (int64_t)T * HS, HS, (int64_t)G * max_seq * HS, (int64_t)max_seq * HS, HS,
                                  (int64_t)G * max_seq * HS, (int64_t)max_seq * HS, HS, (int64_t)T * H * HS, (int64_t)H * HS, nullptr, 0, nullptr, 0,
                                  nullptr, 0, nullptr, 0, 0, nullptr, 0, 0, 0, 0};
  const size_t tiles = (size_t)(kPfBM + 4 * kPfBN) * HS * 2 + (size_t)(kPfBM + 2 * kPfBN) * HK2 * 2;
  const size_t smem = tiles + (size_t)vw.bias_n * sizeof(float);
  static PerDeviceOnce once;
  if (once.need()) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HS, PosT, HK2, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(tiles + kPfBiasTabMax * sizeof(float)));
    if (e != cudaSuccess) return e;
    once.done();
  }
  dim3 grid((T + kPfBM - 1) / kPfBM, H, B);
  return launch(attn_prefill_kernel<HS, PosT, HK2, MODE>, grid, dim3(kPfThreads), smem, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                (const __nv_bfloat16*)vc, (const PosT*)pos, (__nv_bfloat16*)y, T, H, G, max_seq, scale * 1.4426950408889634f, vw);
}

// s'[h] = sum_g talk[h, g] s[g] at every element of the score planes' tiles that the first pass wrote, in place.  The planes share
// one layout, so the same offset in every plane is the same (query row, key) pair: a thread owns an offset, holds its HT >= n_head
// scores in registers and reads the mixing matrix from shared memory.  grid (tiles, 8): a block takes the 16 rows x 64 keys of one warp
// of the tile kernels and leaves at once when that warp skipped the tile (its rows lie before the tile's keys, or past the sequence).
template <int HT>
__global__ void __launch_bounds__(256) mix_scores_kernel(float* __restrict__ sbuf, int64_t s_h, int s_qt, int s_kt, const __nv_bfloat16* __restrict__ talk,
                                                          const int4* __restrict__ seqs, int n_head) {
  __shared__ __align__(16) float tm[HT * HT];
  griddep_launch();
  griddep_wait();
  const int kt = (int)blockIdx.x % s_kt, mt = ((int)blockIdx.x / s_kt) % s_qt, b = (int)blockIdx.x / (s_kt * s_qt), w = blockIdx.y;
  const int4 sq = seqs[b];
  const int first = mt * kPfBM + w * 16;                       // the block's first row in its sequence
  if (first >= sq.y) return;
  if (kt * kPfBN > sq.z + min(first + 15, sq.y - 1)) return;   // every key of the tile lies beyond what these rows see
  for (int i = threadIdx.x; i < HT * HT; i += 256) {
    const int h = i / HT, g = i % HT;
    tm[i] = h < n_head && g < n_head ? __bfloat162float(talk[h * n_head + g]) : 0.f;
  }
  __syncthreads();
  float* base = sbuf + (int64_t)blockIdx.x * (kPfBM * kPfBN) + w * 1024 + threadIdx.x;
  for (int k = 0; k < 4; ++k) {
    float* p = base + k * 256;
    float in[HT];
#pragma unroll
    for (int g = 0; g < HT; ++g) in[g] = g < n_head ? p[(int64_t)g * s_h] : 0.f;
    for (int h = 0; h < n_head; ++h) {
      float acc = 0.f;
#pragma unroll
      for (int g = 0; g < HT; g += 4) {
        const float4 t = *reinterpret_cast<const float4*>(tm + h * HT + g);
        acc = fmaf(t.x, in[g], acc); acc = fmaf(t.y, in[g + 1], acc); acc = fmaf(t.z, in[g + 2], acc); acc = fmaf(t.w, in[g + 3], acc);
      }
      p[(int64_t)h * s_h] = acc;
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

// Causal attention over cache rows with the heads' scores mixed before the softmax, for bf16 prompts on the tensor-core tiles, as
// three launches over fp32 score planes: (1) raw scores of every visible tile, (2) the mixing, in place, (3) softmax with the sink and
// the value product reading the mixed scores back.  sbuf holds n_head planes of n_seqs * ceil(max_q_len / 128) * (s_ld / 64) tiles of
// 8192 floats.  seqs[b] = {first row, rows, first position, cache slot}; k_cache / v_cache rows of a slot are max_seq apart; talk NULL:
// no mixing.
extern "C" size_t b200_attn_prefill_mixed_plane_floats(int n_seqs, int max_q_len, int64_t s_ld) {
  return (size_t)n_seqs * (size_t)((max_q_len + kPfBM - 1) / kPfBM) * (size_t)(s_ld / kPfBN) * (kPfBM * kPfBN);
}

extern "C" int b200_attn_prefill_mixed(const void* q, int64_t ldq, const void* k_cache, int64_t ldk, const void* v_cache, int64_t ldv,
                                       const int32_t* seqs, int n_seqs, int max_q_len, int max_seq, const void* talk, const void* sink, void* y,
                                       int64_t ldy, int n_head, int n_kv_head, int head_size, float scale, float* sbuf, int64_t s_ld,
                                       b200_stream_t stream) {
  B200_CHECK_ARG(q && k_cache && v_cache && seqs && y && sbuf, "b200_attn_prefill_mixed: null pointer");
  B200_CHECK_ARG(n_seqs > 0 && n_seqs <= 65535 && max_q_len > 0 && n_head > 0 && n_head <= 64 && n_kv_head > 0 && n_head % n_kv_head == 0 && max_seq > 0 &&
                     s_ld > 0, "b200_attn_prefill_mixed: bad shape (at most 64 heads)");
  B200_CHECK_ARG(head_size == 64 || head_size == 128, "b200_attn_prefill_mixed: head_size must be 64 or 128 (got %d)", head_size);
  B200_CHECK_ARG(((ldq | ldk | ldv) & 7) == 0 && (ldy & 1) == 0 && (s_ld & 63) == 0, "b200_attn_prefill_mixed: leading dimensions must be multiples of 8 elements, the context bound of 64");
  B200_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                   reinterpret_cast<uintptr_t>(seqs) | reinterpret_cast<uintptr_t>(sbuf)) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 3) == 0,
                 "b200_attn_prefill_mixed: operands must be 16-byte aligned");
  const int s_qt = (max_q_len + kPfBM - 1) / kPfBM, s_kt = (int)(s_ld / kPfBN);
  const int64_t s_h = (int64_t)b200_attn_prefill_mixed_plane_floats(n_seqs, max_q_len, s_ld);
  B200_CHECK_ARG((int64_t)n_seqs * s_qt * s_kt <= 0x7fffffff, "b200_attn_prefill_mixed: too many tiles");
  const PfView vw{0, head_size, ldq, 0, head_size, ldk, 0, head_size, ldv, 0, ldy, reinterpret_cast<const int4*>(seqs), 0,
                  reinterpret_cast<const __nv_bfloat16*>(sink), 0, nullptr, 0, nullptr, 0, 0, sbuf, s_h, s_qt, s_kt, max_seq};
  cudaStream_t st = (cudaStream_t)stream;
  if (head_size == 128) B200_CUDA((launch_prefill<128, int32_t, 0, 1>(q, k_cache, v_cache, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, scale, st, &vw)));
  else B200_CUDA((launch_prefill<64, int32_t, 0, 1>(q, k_cache, v_cache, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, scale, st, &vw)));
  if (talk) {
    const dim3 grid((unsigned)(n_seqs * s_qt * s_kt), 8);
    const __nv_bfloat16* tk = reinterpret_cast<const __nv_bfloat16*>(talk);
    const int4* sq = reinterpret_cast<const int4*>(seqs);
    if (n_head <= 8) B200_CUDA(launch(mix_scores_kernel<8>, grid, dim3(256), 0, st, sbuf, s_h, s_qt, s_kt, tk, sq, n_head));
    else if (n_head <= 16) B200_CUDA(launch(mix_scores_kernel<16>, grid, dim3(256), 0, st, sbuf, s_h, s_qt, s_kt, tk, sq, n_head));
    else if (n_head <= 32) B200_CUDA(launch(mix_scores_kernel<32>, grid, dim3(256), 0, st, sbuf, s_h, s_qt, s_kt, tk, sq, n_head));
    else B200_CUDA(launch(mix_scores_kernel<64>, grid, dim3(256), 0, st, sbuf, s_h, s_qt, s_kt, tk, sq, n_head));
  }
  // the planes are in the log2 domain already: the last pass scales by 1
  if (head_size == 128) B200_CUDA((launch_prefill<128, int32_t, 0, 2>(q, k_cache, v_cache, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, 0.6931471805599453f, st, &vw)));
  else B200_CUDA((launch_prefill<64, int32_t, 0, 2>(q, k_cache, v_cache, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, 0.6931471805599453f, st, &vw)));
  return B200_OK;
}

extern "C" int b200_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const void* pos, int pos_is_int64, void* y,
                                 int batch, int T, int n_head, int n_groups, int head_size, int max_seq, float scale,
                                 b200_stream_t stream) {
  B200_CHECK_ARG(q && k_cache && v_cache && pos && y, "b200_attn_prefill: null pointer");
  B200_CHECK_ARG(batch > 0 && T > 0 && n_head > 0 && n_groups > 0 && max_seq > 0, "b200_attn_prefill: bad shape");
  B200_CHECK_ARG(n_head % n_groups == 0, "b200_attn_prefill: n_head not divisible by n_groups");
  B200_CHECK_ARG(head_size == 64 || head_size == 128, "b200_attn_prefill: head_size must be 64 or 128 (got %d)", head_size);
  B200_CHECK_ARG(n_head <= 65535 && batch <= 65535, "b200_attn_prefill: grid too large");
  cudaStream_t st = (cudaStream_t)stream;
  if (head_size == 128) {
    if (pos_is_int64) B200_CUDA((launch_prefill<128, int64_t>(q, k_cache, v_cache, pos, y, batch, T, n_head, n_groups, max_seq, scale, st)));
    else B200_CUDA((launch_prefill<128, int32_t>(q, k_cache, v_cache, pos, y, batch, T, n_head, n_groups, max_seq, scale, st)));
  } else {
    if (pos_is_int64) B200_CUDA((launch_prefill<64, int64_t>(q, k_cache, v_cache, pos, y, batch, T, n_head, n_groups, max_seq, scale, st)));
    else B200_CUDA((launch_prefill<64, int32_t>(q, k_cache, v_cache, pos, y, batch, T, n_head, n_groups, max_seq, scale, st)));
  }
  return B200_OK;
}

// Ragged batch without rotation or cache layout: packed q (rows, H * hs), k and v (context rows, H * hs) each with its own leading
// dimension (they may be column slices of one buffer), seqs[n_seqs][4] as in PfView, y (rows, H * hs).  One head per key-value head.
extern "C" int b200_attn_prefill_ragged(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                                        int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int head_size, float scale,
                                        b200_stream_t stream) {
  B200_CHECK_ARG(q && k && v && seqs && y, "b200_attn_prefill_ragged: null pointer");
  B200_CHECK_ARG(n_seqs > 0 && n_seqs <= 65535 && max_q_len > 0 && n_head > 0 && n_head <= 65535, "b200_attn_prefill_ragged: bad shape");
  B200_CHECK_ARG(head_size == 64 || head_size == 128, "b200_attn_prefill_ragged: head_size must be 64 or 128 (got %d)", head_size);
  B200_CHECK_ARG(((ldq | ldk | ldv) & 7) == 0 && (ldy & 1) == 0, "b200_attn_prefill_ragged: leading dimensions must be multiples of 8 elements");
  B200_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(seqs)) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(y) & 3) == 0, "b200_attn_prefill_ragged: operands must be 16-byte aligned");
  const PfView vw{0, head_size, ldq, 0, head_size, ldk, 0, head_size, ldv, 0, ldy, reinterpret_cast<const int4*>(seqs), 0, nullptr, 0,
                  nullptr, 0, nullptr, 0, 0, nullptr, 0, 0, 0, 0};
  cudaStream_t st = (cudaStream_t)stream;
  if (head_size == 128) B200_CUDA((launch_prefill<128, int32_t>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  else B200_CUDA((launch_prefill<64, int32_t>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  return B200_OK;
}

// The same tiles for sequences that START in this step (every seqs[b] at position 0): sliding window, sink logits and grouped
// key-value heads; q (rows, H * hs), k and v (rows, G * hs) are the step's own packed rows, seqs[b] = {first row, rows, 0, any}.
extern "C" int b200_attn_prefill_window(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                                        int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int n_kv_head, int head_size, float scale,
                                        int window, const void* sink, b200_stream_t stream) {
  return b200_attn_prefill_window_ex(q, ldq, k, ldk, v, ldv, seqs, n_seqs, max_q_len, y, ldy, n_head, n_kv_head, head_size, scale, window, sink,
                                     nullptr, nullptr, nullptr, 0, 0, stream);
}

extern "C" int b200_attn_prefill_window_ex(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                                           int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int n_kv_head, int head_size, float scale,
                                           int window, const void* sink, const void* r1, const void* r2, const void* gate, int64_t ldg,
                                           int gate_mode, b200_stream_t stream) {
  B200_CHECK_ARG(q && k && v && seqs && y, "b200_attn_prefill_window: null pointer");
  B200_CHECK_ARG(!r1 == !r2 && gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0 || gate), "b200_attn_prefill_window: bad distance bias or gate");
  B200_CHECK_ARG(n_seqs > 0 && n_seqs <= 65535 && max_q_len > 0 && n_head > 0 && n_head <= 65535 && n_kv_head > 0 && n_head % n_kv_head == 0 &&
                 window >= 0, "b200_attn_prefill_window: bad shape");
  B200_CHECK_ARG(head_size == 64 || head_size == 128, "b200_attn_prefill_window: head_size must be 64 or 128 (got %d)", head_size);
  B200_CHECK_ARG(((ldq | ldk | ldv) & 7) == 0 && (ldy & 1) == 0, "b200_attn_prefill_window: leading dimensions must be multiples of 8 elements");
  B200_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(seqs)) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(y) & 3) == 0, "b200_attn_prefill_window: operands must be 16-byte aligned");
  // every visible distance is below the window (or, without one, below the longest sequence of this step, which starts at 0)
  const int reach = window > 0 ? (window < max_q_len ? window : max_q_len) : max_q_len;
  const PfView vw{0, head_size, ldq, 0, head_size, ldk, 0, head_size, ldv, 0, ldy, reinterpret_cast<const int4*>(seqs), window,
                  reinterpret_cast<const __nv_bfloat16*>(sink), 1, nullptr, 0, gate_mode ? reinterpret_cast<const __nv_bfloat16*>(gate) : nullptr, ldg,
                  gate_mode, nullptr, 0, 0, 0, 0, reinterpret_cast<const __nv_bfloat16*>(r1), reinterpret_cast<const __nv_bfloat16*>(r2),
                  r1 && reach <= kPfBiasTabMax ? reach : 0};
  cudaStream_t st = (cudaStream_t)stream;
  if (head_size == 128) B200_CUDA((launch_prefill<128, int32_t>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, scale, st, &vw)));
  else B200_CUDA((launch_prefill<64, int32_t>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_kv_head, 0, scale, st, &vw)));
  return B200_OK;
}

// The ragged tiles for latent attention with a key part shared by the heads: q (rows, H * (hs + dk2)) with each head laid out as
// [hs | dk2]; k, v (context rows, H * hs) expanded per head; k2 (context rows, dk2) the shared part; optional sink logits and a
// sigmoid output gate (gate_mode 1: one column per head, 2: one per output number).  hs in {64, 128}, dk2 in {64, 128}.
extern "C" int b200_attn_prefill_shared(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* k2,
                                        int64_t ldk2, int dk2, const int32_t* seqs, int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head,
                                        int head_size, float scale, const void* sink, const void* gate, int64_t ldg, int gate_mode,
                                        b200_stream_t stream) {
  B200_CHECK_ARG(q && k && v && k2 && seqs && y, "b200_attn_prefill_shared: null pointer");
  B200_CHECK_ARG(n_seqs > 0 && n_seqs <= 65535 && max_q_len > 0 && n_head > 0 && n_head <= 65535, "b200_attn_prefill_shared: bad shape");
  B200_CHECK_ARG((head_size == 64 || head_size == 128) && (dk2 == 64 || dk2 == 128), "b200_attn_prefill_shared: sizes must be 64 or 128 (got %d, %d)",
                 head_size, dk2);
  B200_CHECK_ARG(gate_mode >= 0 && gate_mode <= 2 && (gate_mode == 0 || gate), "b200_attn_prefill_shared: bad gate");
  B200_CHECK_ARG(((ldq | ldk | ldv | ldk2) & 7) == 0 && (ldy & 1) == 0, "b200_attn_prefill_shared: leading dimensions must be multiples of 8 elements");
  B200_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(k2) |
                   reinterpret_cast<uintptr_t>(seqs)) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 3) == 0,
                 "b200_attn_prefill_shared: operands must be 16-byte aligned");
  const PfView vw{0, head_size + dk2, ldq, 0, head_size, ldk, 0, head_size, ldv, 0, ldy, reinterpret_cast<const int4*>(seqs), 0,
                  reinterpret_cast<const __nv_bfloat16*>(sink), 0, reinterpret_cast<const __nv_bfloat16*>(k2), ldk2,
                  reinterpret_cast<const __nv_bfloat16*>(gate), ldg, gate_mode, nullptr, 0, 0, 0, 0};
  cudaStream_t st = (cudaStream_t)stream;
  if (head_size == 128 && dk2 == 64) B200_CUDA((launch_prefill<128, int32_t, 64>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  else if (head_size == 128) B200_CUDA((launch_prefill<128, int32_t, 128>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  else if (dk2 == 64) B200_CUDA((launch_prefill<64, int32_t, 64>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  else B200_CUDA((launch_prefill<64, int32_t, 128>(q, k, v, nullptr, y, n_seqs, max_q_len, n_head, n_head, 0, scale, st, &vw)));
  return B200_OK;
}
