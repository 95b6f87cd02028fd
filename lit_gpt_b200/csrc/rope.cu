// Per-head preparation of projected rows before attention: an optional weighted RMS norm over the head, rotary positions on a
// run of its dimensions, and the move to where the attention reads it -- in place, to a dense buffer, or scattered into the
// rows of a cache.
//
//   z = head / sqrt(mean(head^2) + eps) * w                    (optional; statistics over the whole head, fp32)
//   (u, v) <- (u cos a - v sin a, v cos a + u sin a) * mag     for the pairs of dimensions [rot_off, rot_off + rot_dims):
//             pair i = (2 i, 2 i + 1) when interleaved, else (i, i + rot_dims / 2); a = position * freq[i] in fp32
//   the other dimensions pass unchanged.
//
// Up to three groups of heads (e.g. queries, keys, values of one fused projection) run as one launch; one warp per (row, head).
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

template <typename T>
__global__ void __launch_bounds__(kHrThreads) head_rope_kernel(HeadSegs S, const int* __restrict__ row_pos, int64_t rows, float eps) {
  griddep_launch();
  griddep_wait();
  const HeadSeg s = S.s[blockIdx.y];
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * (kHrThreads / 32) + (threadIdx.x >> 5);
  if (item >= rows * s.heads) return;
  const int64_t row = item / s.heads;
  const int h = (int)(item - row * s.heads);
  const int64_t orow = s.out_rows ? s.out_rows[row] : row;
  if (orow < 0) return;
  const T* x = reinterpret_cast<const T*>(s.in) + row * s.ld_in + (int64_t)h * s.in_stride;
  T* o = reinterpret_cast<T*>(s.out) + orow * s.ld_out + (int64_t)h * s.out_stride;
  const T* w = reinterpret_cast<const T*>(s.norm_w);
  float rstd = 1.0f;
  if (w) {
    float ss = 0.f;
    for (int i = lane; i < s.dim; i += 32) { const float v = load_as_float(x, i); ss = fmaf(v, v, ss); }
    rstd = 1.0f / sqrtf(warp_sum(ss) / (float)s.dim + eps);   // the shuffle also orders every lane's reads before any write below
  }
  const int half = s.rot_dims / 2;
  const float pos = (float)row_pos[row];
  // the rotated pairs: both members are read before either is written, and no other lane touches them
  for (int i = lane; i < half; i += 32) {
    const int a = s.rot_off + (s.interleaved ? 2 * i : i), b = s.rot_off + (s.interleaved ? 2 * i + 1 : i + half);
    float u = load_as_float(x, a), v = load_as_float(x, b);
    if (w) { u = u * rstd * load_as_float(w, a); v = v * rstd * load_as_float(w, b); }
    float sn, cs;
    sincosf(pos * s.freq[i], &sn, &cs);
    sn *= s.mag; cs *= s.mag;
    store_from_float(o, a, u * cs - v * sn);
    store_from_float(o, b, v * cs + u * sn);
  }
  const bool moved = (const void*)o != (const void*)x;
  if (!w && !moved) return;
  for (int i = lane; i < s.dim; i += 32) {
    if (i >= s.rot_off && i < s.rot_off + 2 * half) continue;
    float v = load_as_float(x, i);
    if (w) v = v * rstd * load_as_float(w, i);
    store_from_float(o, i, v);
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
  int max_heads = 0;
  for (int i = 0; i < kHrMaxSegs; ++i) {
    const b200_head_rope_seg& a = segs[i < n_segs ? i : 0];
    B200_CHECK_ARG(a.in && a.out && a.heads > 0 && a.dim > 0, "b200_head_rope: null pointer or empty head");
    B200_CHECK_ARG(a.rot_dims >= 0 && a.rot_dims % 2 == 0 && a.rot_off >= 0 && a.rot_off + a.rot_dims <= a.dim && (a.rot_dims == 0 || a.freq),
                   "b200_head_rope: the rotated dimensions must be an even run inside the head, with their frequencies");
    S.s[i] = HeadSeg{a.in, a.out, a.norm_w, a.freq, a.out_rows, a.ld_in, a.ld_out, a.heads, a.dim, a.in_stride, a.out_stride, a.rot_off, a.rot_dims,
                     a.interleaved, a.mag};
    if (i < n_segs) max_heads = a.heads > max_heads ? a.heads : max_heads;
  }
  const int64_t blocks = (rows * max_heads + kHrThreads / 32 - 1) / (kHrThreads / 32);
  B200_CHECK_ARG(blocks <= 0x7fffffff, "b200_head_rope: too many rows");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(head_rope_kernel<T>, dim3((unsigned)blocks, (unsigned)n_segs), dim3(kHrThreads), 0, (cudaStream_t)stream, S,
                                               row_pos, rows, eps)));
  return B200_OK;
}

}  // extern "C"
