// Sliding-window attention with an attention sink, over a ring of cached keys and values.
//
//   row at position i sees positions j with 0 <= i - j < window;  p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j')),
//   s_j = (q . k_j) * scale.  The sink is one learned logit per head with no key and no value: it only takes probability.
//   Optional: a distance bias, s_j -= r1_h * ln(1 + r2_h * (i - j)) with two numbers per head, and a sigmoid output gate read from
//   raw projections of the row (one per head, or one per output number).
//
// Grouped heads (query head h reads key-value head h / (H / G)), separate query-key (dk) and value (dv) sizes, any sizes,
// operands bf16 or fp32, all arithmetic fp32 with a running maximum.
//
// Only the last `ring` >= window positions of a sequence are kept: position p lives in row p % ring of the sequence's slot.
// A step's own keys and values are read from the step's packed rows (k, v), older ones from the ring, so one kernel serves
// a whole prompt, a later portion of one and single decoded tokens; the step's last rows enter the ring AFTERWARDS (a long
// step would otherwise overwrite ring rows that its first queries still need): b200_ring_store after the tiled kernel, the
// single-row kernel itself for its one row.
//
//  * window_attn_kernel: 64 query rows x 64 keys per tile (the shape of latent_prefill_kernel), for steps with many rows.
//  * window_decode_kernel: one CTA per (sequence, head) for single rows: scores of the whole window in shared memory, one
//    pass for the softmax, then the value sum with the window split over thread rows; 16-byte loads where the operands allow.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kWaBM = 64, kWaBN = 64, kWaDV = 128, kWaThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

__host__ __device__ inline int wa_pitch(int d) {   // a multiple of 4 with pitch / 4 odd: float4 reads of rows one apart do not collide
  int p = (d + 3) & ~3;
  if (((p >> 2) & 1) == 0) p += 4;
  return p;
}

struct WaArgs {
  const void* q; const void* k; const void* v; void* out;
  int64_t ldq, ldk, ldv, ldo;
  const void* k_ring; const void* v_ring;
  const void* sink;
  const int4* seqs;
  int ring, n_head, n_kv_head, dk, dv, window;
  float scale_log2;
  int store_ring;
  const void* r1; const void* r2;   // distance bias per head (NULL: none)
  const void* gate;                 // raw gate projections, rows ldg apart (NULL: none)
  int64_t ldg;
  int gate_mode;                    // 1: column h of the gate row; 2: column h * dv + c
};

// output gate of one number: sigmoid of the raw projection
template <typename T>
__device__ __forceinline__ float wa_gate(const WaArgs& A, int64_t row, int h, int c) {
  if (!A.gate) return 1.0f;
  const float z = load_as_float(reinterpret_cast<const T*>(A.gate), row * A.ldg + (A.gate_mode == 1 ? h : (int64_t)h * A.dv + c));
  return 1.0f / (1.0f + expf(-z));
}

template <typename T>
__global__ void __launch_bounds__(kWaThreads) window_attn_kernel(WaArgs A) {
  extern __shared__ __align__(16) float wa_smem[];
  griddep_launch();
  griddep_wait();
  const T* const q = reinterpret_cast<const T*>(A.q);
  const T* const k = reinterpret_cast<const T*>(A.k);
  const T* const v = reinterpret_cast<const T*>(A.v);
  const T* const kr = reinterpret_cast<const T*>(A.k_ring);
  const T* const vr = reinterpret_cast<const T*>(A.v_ring);
  const int4 sq = A.seqs[blockIdx.z];
  const int first = sq.x, qlen = sq.y, pos0 = sq.z, slot = sq.w;
  const int r0 = (int)blockIdx.x * kWaBM;
  if (r0 >= qlen) return;
  const int dk = A.dk, dv = A.dv, G = A.n_kv_head;
  const int nchunk = (dv + kWaDV - 1) / kWaDV;
  const int h = (int)blockIdx.y / nchunk, c0 = ((int)blockIdx.y % nchunk) * kWaDV;
  const int g = h / (A.n_head / G);
  const int dvc = min(kWaDV, dv - c0);
  const int dkp = wa_pitch(dk);
  constexpr int PP = kWaBN + 4;
  float* const Qs = wa_smem;                          // [64][dkp]
  float* const Ks = Qs + kWaBM * dkp;                 // [64][dkp]
  float* const Vs = Ks + kWaBN * dkp;                 // [64][128]
  float* const Ps = Vs + kWaBN * kWaDV;               // [64][68]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  for (int idx = tid; idx < kWaBM * dkp; idx += kWaThreads) {
    const int i = idx / dkp, d = idx - i * dkp;
    float val = 0.f;
    if (r0 + i < qlen && d < dk) val = load_as_float(q, (int64_t)(first + r0 + i) * A.ldq + (int64_t)h * dk + d) * A.scale_log2;
    Qs[idx] = val;
  }
  const int last_row = min(r0 + kWaBM, qlen) - 1;
  const int key_hi = pos0 + last_row + 1;                       // one past the last visible key
  const int key_lo = max(0, pos0 + r0 - A.window + 1);           // first key the tile's first row sees

  float o[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) o[a][b] = 0.f;
  float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l_run[4] = {0.f, 0.f, 0.f, 0.f};
  int lim[4];                                                   // position of each of this thread's rows (-1: no row)
#pragma unroll
  for (int a = 0; a < 4; ++a) lim[a] = (r0 + ty + 16 * a < qlen) ? pos0 + r0 + ty + 16 * a : -1;
  // scores live in the log2 domain: r1 ln(1 + r2 dist) log2(e) = r1 log2(1 + r2 dist)
  const bool biased = A.r1 != nullptr;
  const float r1h = biased ? load_as_float(reinterpret_cast<const T*>(A.r1), h) : 0.f;
  const float r2h = biased ? load_as_float(reinterpret_cast<const T*>(A.r2), h) : 0.f;

  for (int j0 = key_lo; j0 < key_hi; j0 += kWaBN) {
    __syncthreads();
    for (int idx = tid; idx < kWaBN * dkp; idx += kWaThreads) {
      const int j = idx / dkp, d = idx - j * dkp;
      const int p = j0 + j;
      float val = 0.f;
      if (p < key_hi && d < dk)
        val = p >= pos0 ? load_as_float(k, (int64_t)(first + p - pos0) * A.ldk + (int64_t)g * dk + d)
                        : load_as_float(kr, ((int64_t)slot * A.ring + p % A.ring) * G * dk + (int64_t)g * dk + d);
      Ks[idx] = val;
    }
    for (int idx = tid; idx < kWaBN * kWaDV; idx += kWaThreads) {
      const int j = idx / kWaDV, c = idx - j * kWaDV;
      const int p = j0 + j;
      float val = 0.f;
      if (p < key_hi && c < dvc)
        val = p >= pos0 ? load_as_float(v, (int64_t)(first + p - pos0) * A.ldv + (int64_t)g * dv + c0 + c)
                        : load_as_float(vr, ((int64_t)slot * A.ring + p % A.ring) * G * dv + (int64_t)g * dv + c0 + c);
      Vs[idx] = val;
    }
    __syncthreads();

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
    float alpha[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float mx = -INFINITY;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int p = j0 + tx + 16 * b;
        if (p > lim[a] || p <= lim[a] - A.window) s[a][b] = -INFINITY;   // ahead of the row, or fallen out of its window
        else if (biased) s[a][b] -= r1h * log2f(fmaf(r2h, (float)(lim[a] - p), 1.0f));
        mx = fmaxf(mx, s[a][b]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[a], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[a] = exp2f(m_run[a] - m_safe);
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
    for (int j = 0; j < kWaBN; j += 4) {
      float4 pa[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) pa[a] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * a) * PP + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 v0 = *reinterpret_cast<const float4*>(Vs + (j + jj) * kWaDV + 4 * tx);
        const float4 v1 = *reinterpret_cast<const float4*>(Vs + (j + jj) * kWaDV + 64 + 4 * tx);
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
  const float sink_l2 = A.sink ? load_as_float(reinterpret_cast<const T*>(A.sink), h) * kLog2e : -INFINITY;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = r0 + ty + 16 * a;
    if (i >= qlen) continue;
    // the sink joins the denominator once, unscaled
    const float m_fin = fmaxf(m_run[a], sink_l2);
    const float c = exp2f(m_run[a] - m_fin);
    const float inv = c / (l_run[a] * c + exp2f(sink_l2 - m_fin));
    T* orow = reinterpret_cast<T*>(A.out) + (int64_t)(first + i) * A.ldo + (int64_t)h * dv + c0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int cc = (b < 4 ? 0 : 64) + 4 * tx + (b & 3);
      if (cc < dvc) store_from_float(orow, cc, o[a][b] * inv * wa_gate<T>(A, first + i, h, c0 + cc));
    }
  }
}

// One row per sequence.  grid (n_head, n_seqs), 256 threads.  Scores for the whole window sit in shared memory.
// VEC (every row of q, k, v and the rings starts on a 16-byte boundary and dk, dv are multiples of 8): eight lanes share one
// key and read it in 8-element pieces, so a warp takes four keys per pass; for the value sum a thread owns eight neighbouring
// columns and the window is split over the 256 / (dv / 8) thread rows, whose partial sums are added in a fixed order.
constexpr int kWdThreads = 256, kWdWarps = kWdThreads / 32;

__host__ __device__ inline int wd_value_rows(int dv, bool vec) { return vec ? kWdThreads / (dv / 8) : kWdWarps; }

template <typename T, bool VEC>
__global__ void __launch_bounds__(kWdThreads) window_decode_kernel(WaArgs A) {
  extern __shared__ __align__(16) float wd_smem[];
  __shared__ float s_red[kWdWarps];
  griddep_launch();
  griddep_wait();
  const int h = blockIdx.x, g = h / (A.n_head / A.n_kv_head), G = A.n_kv_head;
  const int4 sq = A.seqs[blockIdx.y];
  const int row = sq.x, pos = sq.z, slot = sq.w;
  const int dk = A.dk, dv = A.dv;
  const int lo = max(0, pos - A.window + 1), n = pos - lo + 1;     // visible positions lo .. pos
  float* const qs = wd_smem;                        // [dk rounded up to 8]
  float* const sc = qs + ((dk + 7) & ~7);           // [window rounded up to 4]
  float* const part = sc + ((A.window + 3) & ~3);   // [value rows][dv]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* const kr = reinterpret_cast<const T*>(A.k_ring);
  const T* const vr = reinterpret_cast<const T*>(A.v_ring);
  const T* const k_now = reinterpret_cast<const T*>(A.k) + (int64_t)row * A.ldk + (int64_t)g * dk;
  const T* const v_now = reinterpret_cast<const T*>(A.v) + (int64_t)row * A.ldv + (int64_t)g * dv;
  auto key_row = [&](int p) { return p == pos ? k_now : kr + ((int64_t)slot * A.ring + p % A.ring) * G * dk + (int64_t)g * dk; };
  auto value_row = [&](int p) { return p == pos ? v_now : vr + ((int64_t)slot * A.ring + p % A.ring) * G * dv + (int64_t)g * dv; };
  for (int d = tid; d < dk; d += kWdThreads) qs[d] = load_as_float(reinterpret_cast<const T*>(A.q), (int64_t)row * A.ldq + (int64_t)h * dk + d) * A.scale_log2;
  __syncthreads();
  float mx = -INFINITY;
  // distance bias in the log2 domain; visible position j of n lies n - 1 - j behind the row
  const bool biased = A.r1 != nullptr;
  const float r1h = biased ? load_as_float(reinterpret_cast<const T*>(A.r1), h) : 0.f;
  const float r2h = biased ? load_as_float(reinterpret_cast<const T*>(A.r2), h) : 0.f;
  if (VEC) {
    const int sub = tid & 7, grp = tid >> 3;          // 32 groups of eight lanes, one key each per pass
    constexpr int KG = kWdThreads / 8, U = 4;         // four passes' loads are issued before any of them is used
    for (int jb = 0; jb < n; jb += KG * U) {
      float acc[U];
      if (dk <= 128) {
        float f[U][2][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = jb + u * KG + grp;
          const T* kp = key_row(lo + min(j, n - 1));
#pragma unroll
          for (int pc = 0; pc < 2; ++pc) {
            const int c = sub * 8 + pc * 64;
            if (j < n && c < dk) load8(kp + c, f[u][pc]);
            else {
#pragma unroll
              for (int e = 0; e < 8; ++e) f[u][pc][e] = 0.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          acc[u] = 0.f;
#pragma unroll
          for (int pc = 0; pc < 2; ++pc) {
            const int c = sub * 8 + pc * 64;
            if (c < dk) {
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[u] = fmaf(qs[c + e], f[u][pc][e], acc[u]);
            }
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = jb + u * KG + grp;
          acc[u] = 0.f;
          if (j < n) {
            const T* kp = key_row(lo + j);
            for (int c = sub * 8; c < dk; c += 64) {
              float f[8];
              load8(kp + c, f);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[u] = fmaf(qs[c + e], f[e], acc[u]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = jb + u * KG + grp;
        float a = acc[u];
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        if (j < n) {
          if (biased) a -= r1h * log2f(fmaf(r2h, (float)(n - 1 - j), 1.0f));
          if (sub == 0) sc[j] = a;
          mx = fmaxf(mx, a);
        }
      }
    }
  } else {
    for (int j = warp; j < n; j += kWdWarps) {       // one warp per key
      const T* kp = key_row(lo + j);
      float acc = 0.f;
      for (int d = lane; d < dk; d += 32) acc = fmaf(qs[d], load_as_float(kp, d), acc);
      acc = warp_sum(acc);
      if (biased) acc -= r1h * log2f(fmaf(r2h, (float)(n - 1 - j), 1.0f));
      if (lane == 0) sc[j] = acc;
      mx = fmaxf(mx, acc);
    }
  }
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = s_red[0];
#pragma unroll
  for (int w = 1; w < kWdWarps; ++w) mx = fmaxf(mx, s_red[w]);
  const float sink_l2 = A.sink ? load_as_float(reinterpret_cast<const T*>(A.sink), h) * kLog2e : -INFINITY;
  mx = fmaxf(mx, sink_l2);
  float sum = 0.f;
  for (int j = tid; j < n; j += kWdThreads) {
    const float p = exp2f(sc[j] - mx);
    sc[j] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncthreads();                      // s_red read by everyone above
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();                      // also: every probability is in shared memory
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kWdWarps; ++w) total += s_red[w];
  const float inv = 1.0f / (total + exp2f(sink_l2 - mx));   // the sink joins the denominator once, unscaled
  const int vrows = wd_value_rows(dv, VEC);
  if (VEC) {
    const int ncg = dv / 8, cg = tid % ncg, rj = tid / ncg;
    if (rj < vrows) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int j = rj; j < n; j += vrows) {
        float f[8];
        load8(value_row(lo + j) + cg * 8, f);
        const float p = sc[j];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(p, f[e], acc[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) part[rj * dv + cg * 8 + e] = acc[e];
    }
  } else {
    for (int c = lane; c < dv; c += 32) {
      float acc = 0.f;
      for (int j = warp; j < n; j += kWdWarps) acc = fmaf(sc[j], load_as_float(value_row(lo + j), c), acc);
      part[warp * dv + c] = acc;
    }
  }
  __syncthreads();
  for (int c = tid; c < dv; c += kWdThreads) {
    float t = 0.f;
    for (int r = 0; r < vrows; ++r) t += part[r * dv + c];
    store_from_float(reinterpret_cast<T*>(A.out), (int64_t)row * A.ldo + (int64_t)h * dv + c, t * inv * wa_gate<T>(A, row, h, c));
  }
  // The row's own key and value enter the ring here: they replace position pos - ring, which no row of this step can see
  // (ring >= window), and every CTA reads the current position from the step's rows, never from the ring.
  if (A.store_ring && h % (A.n_head / G) == 0) {
    T* kd = const_cast<T*>(kr) + ((int64_t)slot * A.ring + pos % A.ring) * G * dk + (int64_t)g * dk;
    T* vd = const_cast<T*>(vr) + ((int64_t)slot * A.ring + pos % A.ring) * G * dv + (int64_t)g * dv;
    for (int d = tid; d < dk; d += kWdThreads) kd[d] = k_now[d];
    for (int c = tid; c < dv; c += kWdThreads) vd[c] = v_now[c];
  }
}

// ring[slot][p % ring] <- row, for the rows whose position p is among the sequence's last `ring`
template <typename T>
__global__ void __launch_bounds__(128) ring_store_kernel(const T* __restrict__ k, int64_t ldk, const T* __restrict__ v, int64_t ldv,
                                                         T* __restrict__ k_ring, T* __restrict__ v_ring, int ring, int kcols, int vcols,
                                                         const int4* __restrict__ seqs, const int* __restrict__ row_seq) {
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  const int4 sq = seqs[row_seq[row]];
  const int p = sq.z + (int)(row - sq.x), end = sq.z + sq.y;
  if (p < end - ring) return;
  const int64_t dst = (int64_t)sq.w * ring + p % ring;
  for (int i = threadIdx.x; i < kcols; i += 128) k_ring[dst * kcols + i] = k[row * ldk + i];
  for (int i = threadIdx.x; i < vcols; i += 128) v_ring[dst * vcols + i] = v[row * ldv + i];
}

int g_wa_force_tiled = 0;

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_window_attn_tune(int force_tiled_kernel) {
  const int old = g_wa_force_tiled;
  g_wa_force_tiled = force_tiled_kernel ? 1 : 0;
  return old;
}

int b200_window_attn(const b200_window_attn_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->q && a->k && a->v && a->out && a->seqs, "b200_window_attn: null pointer");
  B200_CHECK_ARG(a->n_seqs > 0 && a->n_seqs <= 65535 && a->max_q_len > 0, "b200_window_attn: bad batch");
  B200_CHECK_ARG(a->n_head > 0 && a->n_kv_head > 0 && a->n_head % a->n_kv_head == 0 && a->dk > 0 && a->dk <= 512 && a->dv > 0,
                 "b200_window_attn: bad head shape (query-key size up to 512)");
  B200_CHECK_ARG(a->window > 0 && a->ring >= a->window && a->k_ring && a->v_ring, "b200_window_attn: the ring must hold at least one window");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(a->seqs) & 15) == 0, "b200_window_attn: seqs must be 16-byte aligned");
  B200_CHECK_ARG(!a->dist_r1 == !a->dist_r2, "b200_window_attn: the distance bias needs both of its numbers per head");
  B200_CHECK_ARG(a->gate_mode >= 0 && a->gate_mode <= 2 && (a->gate_mode == 0 || a->gate), "b200_window_attn: bad gate");
  const WaArgs A{a->q, a->k, a->v, a->out, a->ldq, a->ldk, a->ldv, a->ldo, a->k_ring, a->v_ring, a->sink, reinterpret_cast<const int4*>(a->seqs),
                 a->ring, a->n_head, a->n_kv_head, a->dk, a->dv, a->window, a->scale * kLog2e, a->row_seq != nullptr,
                 a->dist_r1, a->dist_r2, a->gate_mode ? a->gate : nullptr, a->ldg, a->gate_mode};
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = a->dtype == B200_F32 ? 4 : 2;
  auto aligned = [&](const void* p, int64_t ld) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * esz) % 16 == 0; };
  const bool vec = a->dk % 8 == 0 && a->dv % 8 == 0 && a->dv <= 8 * kWdThreads && aligned(a->k, a->ldk) && aligned(a->v, a->ldv) &&
                   aligned(a->k_ring, 8) && aligned(a->v_ring, 8);
  const size_t smem_d = (size_t)(((a->dk + 7) & ~7) + ((a->window + 3) & ~3) + wd_value_rows(a->dv, vec) * a->dv) * sizeof(float);
  if (a->max_q_len == 1 && !g_wa_force_tiled && smem_d <= 160 * 1024 && a->n_head <= 65535) {
    B200_FLOAT_TYPES(a->dtype, T, {
      static PerDeviceOnce once;
      if (smem_d > 48 * 1024 && once.need()) {
        B200_CUDA(cudaFuncSetAttribute(window_decode_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(window_decode_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        once.done();
      }
      if (vec) B200_CUDA(launch(window_decode_kernel<T, true>, dim3((unsigned)a->n_head, (unsigned)a->n_seqs), dim3(kWdThreads), smem_d, st, A));
      else B200_CUDA(launch(window_decode_kernel<T, false>, dim3((unsigned)a->n_head, (unsigned)a->n_seqs), dim3(kWdThreads), smem_d, st, A));
    });
    return B200_OK;
  }
  const int nchunk = (a->dv + kWaDV - 1) / kWaDV;
  B200_CHECK_ARG((int64_t)a->n_head * nchunk <= 65535, "b200_window_attn: too many heads");
  const size_t smem = (size_t)(2 * kWaBM * wa_pitch(a->dk) + kWaBN * kWaDV + kWaBM * (kWaBN + 4)) * sizeof(float);
  const dim3 grid((unsigned)((a->max_q_len + kWaBM - 1) / kWaBM), (unsigned)(a->n_head * nchunk), (unsigned)a->n_seqs);
  B200_FLOAT_TYPES(a->dtype, T, {
    static PerDeviceOnce once;
    if (once.need()) {
      B200_CUDA(cudaFuncSetAttribute(window_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      once.done();
    }
    B200_CHECK_ARG(smem <= 200 * 1024, "b200_window_attn: head size too large for the tile");
    B200_CUDA(launch(window_attn_kernel<T>, grid, dim3(kWaThreads), smem, st, A));
  });
  if (a->row_seq)
    return b200_ring_store(a->k, a->ldk, a->v, a->ldv, const_cast<void*>(a->k_ring), const_cast<void*>(a->v_ring), a->ring, a->n_kv_head * a->dk,
                           a->n_kv_head * a->dv, a->seqs, a->row_seq, a->rows, a->dtype, stream);
  return B200_OK;
}

int b200_ring_store(const void* k, int64_t ldk, const void* v, int64_t ldv, void* k_ring, void* v_ring, int ring, int kcols, int vcols,
                    const int32_t* seqs, const int32_t* row_seq, int64_t rows, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(k && v && k_ring && v_ring && seqs && row_seq, "b200_ring_store: null pointer");
  B200_CHECK_ARG(ring > 0 && kcols > 0 && vcols > 0 && rows > 0 && rows <= 0x7fffffff, "b200_ring_store: bad shape");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(seqs) & 15) == 0, "b200_ring_store: seqs must be 16-byte aligned");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(ring_store_kernel<T>, dim3((unsigned)rows), dim3(128), 0, (cudaStream_t)stream, (const T*)k, ldk,
                                               (const T*)v, ldv, (T*)k_ring, (T*)v_ring, ring, kcols, vcols, reinterpret_cast<const int4*>(seqs), row_seq)));
  return B200_OK;
}

}  // extern "C"
