// Glue kernels for models that keep the residual stream in fp32 beside a working copy in the matrix-product dtype
// (bf16 or fp32): token + position embedding, RMS norms over strided / gathered / scattered rows (statistics always in
// fp32), the "x += norm(branch)" residual update of post-normed blocks, a row gather and the logit scale.
// One CTA per row; rows are a few hundred to a few thousand elements, so these are launch- and latency-bound.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kRowThreads = 128;

// sum over the CTA (kRowThreads threads); every thread gets the result
__device__ __forceinline__ float cta_sum(float v, float* s_part) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // s_part may still be read from a previous call
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kRowThreads / 32; ++w) t += s_part[w];
  return t;
}

// x[row] = embed[token[row]] * scale + pos_table[pos[row]]  (fp32), act[row] = T(x[row])
template <typename T>
__global__ void __launch_bounds__(kRowThreads) embed_pos_kernel(const int* __restrict__ tokens, const int* __restrict__ pos,
                                                                 const T* __restrict__ embed, const T* __restrict__ pos_table,
                                                                 float scale, float* __restrict__ x, T* __restrict__ act, int d,
                                                                 int vocab, int max_pos) {
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // never read out of bounds
  const T* e = embed + (int64_t)tok * d;
  const T* p = nullptr;
  if (pos_table) {
    int pp = pos[row];
    pp = pp < 0 ? 0 : (pp >= max_pos ? max_pos - 1 : pp);
    p = pos_table + (int64_t)pp * d;
  }
  for (int i = threadIdx.x; i < d; i += kRowThreads) {
    float v = load_as_float(e, i) * scale;
    if (p) v += load_as_float(p, i);
    x[row * d + i] = v;
    store_from_float(act, row * d + i, v);
  }
}

// out[orow] = in[irow] / sqrt(mean(in[irow]^2) + eps) * (weight or 1 + weight); blockIdx.y picks one of two segments so
// that the two norms that follow one fused down-projection run as a single launch
struct RmsSeg {
  const void* in;
  const void* weight;
  void* out;
  const int64_t* in_rows;   // NULL: row index itself
  const int64_t* out_rows;  // NULL: row index itself
  int64_t ld_in, ld_out;
  int d, plus_one;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(kRowThreads) rms_rows_kernel(RmsSeg s0, RmsSeg s1, float eps) {
  __shared__ float s_part[kRowThreads / 32];
  griddep_launch();
  griddep_wait();
  const RmsSeg s = blockIdx.y == 0 ? s0 : s1;
  const int64_t row = blockIdx.x;
  const int64_t irow = s.in_rows ? s.in_rows[row] : row, orow = s.out_rows ? s.out_rows[row] : row;
  if (orow < 0) return;   // a row with nowhere to go (padding)
  const TI* xr = reinterpret_cast<const TI*>(s.in) + irow * s.ld_in;
  const TO* w = reinterpret_cast<const TO*>(s.weight);
  TO* yr = reinterpret_cast<TO*>(s.out) + orow * s.ld_out;
  const bool vec = vec8_ok(s.d, xr, w, yr);
  const float one = s.plus_one ? 1.0f : 0.0f;
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < s.d; i += kRowThreads * 8) {
      float v[8];
      load8(xr + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < s.d; i += kRowThreads) {
      const float v = load_as_float(xr, i);
      ss = fmaf(v, v, ss);
    }
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, s_part) / (float)s.d + eps);
  if (vec) {
    for (int i = threadIdx.x * 8; i < s.d; i += kRowThreads * 8) {
      float v[8], g[8];
      load8(xr + i, v);
      load8(w + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * rstd * (g[j] + one);
      store8(yr + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < s.d; i += kRowThreads) store_from_float(yr, i, load_as_float(xr, i) * rstd * (load_as_float(w, i) + one));
  }
}

// x[row] += y[row] / sqrt(mean(y[row]^2) + eps) * (1 + w);  act[row] = T(x[row]).  x stays fp32.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) residual_norm_add_kernel(const T* __restrict__ y, const T* __restrict__ w, float eps,
                                                                         float* __restrict__ x, T* __restrict__ act, int d) {
  __shared__ float s_part[kRowThreads / 32];
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  const T* yr = y + row * d;
  float* xr = x + row * d;
  T* ar = act + row * d;
  const bool vec = vec8_ok(d, yr, w, xr, ar);
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
      float v[8];
      load8(yr + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) {
      const float v = load_as_float(yr, i);
      ss = fmaf(v, v, ss);
    }
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, s_part) / (float)d + eps);
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
      float v[8], g[8], r[8];
      load8(yr + i, v);
      load8(w + i, g);
      load8(xr + i, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = r[j] + v[j] * rstd * (1.0f + g[j]);
      store8(xr + i, r);
      store8(ar + i, r);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) {
      const float v = xr[i] + load_as_float(yr, i) * rstd * (1.0f + load_as_float(w, i));
      xr[i] = v;
      store_from_float(ar, i, v);
    }
  }
}


// Residual update of a block with norms before AND after each sublayer, fused with the norm that feeds the next sublayer:
//   y    = y0                                   (one branch)
//        | (norm(y0) * w0 + norm(y1) * w1) / 2  (two mixers side by side, each RMS-normed over the width with its own weight)
//   x   += norm(y) * post_w  [+ extra]          (fp32 stream; `extra`: e.g. the embedding re-entering before a repeated pass)
//   act  = T(norm(x) * pre_w)                   (input of the next sublayer; skipped without pre_w)
// norm(z) = z / sqrt(mean(z^2) + eps), statistics in fp32.  One CTA per row; the row lives in shared memory between the passes.
struct SandwichArgs {
  const void* y0; const void* w0; const void* y1; const void* w1;
  const void* post_w; const float* extra; const void* pre_w;
  float* x; void* act;
  int d;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(kRowThreads) sandwich_residual_kernel(SandwichArgs A) {
  extern __shared__ __align__(16) float sw_row[];   // [d]
  __shared__ float s_part[kRowThreads / 32];
  griddep_launch();
  griddep_wait();
  const int64_t row = blockIdx.x;
  const int d = A.d;
  const T* y0 = reinterpret_cast<const T*>(A.y0) + row * d;
  const T* y1 = A.y1 ? reinterpret_cast<const T*>(A.y1) + row * d : nullptr;
  const T* w0 = reinterpret_cast<const T*>(A.w0);
  const T* w1 = reinterpret_cast<const T*>(A.w1);
  const T* pw = reinterpret_cast<const T*>(A.post_w);
  const T* nw = reinterpret_cast<const T*>(A.pre_w);
  float* xr = A.x + row * d;
  const float* ex = A.extra ? A.extra + row * d : nullptr;
  T* ar = nw ? reinterpret_cast<T*>(A.act) + row * d : nullptr;
  // eight elements per access when every row and weight starts on a 16-byte boundary (d a multiple of 8, aligned bases)
  const bool vec = vec8_ok(d, A.y0, A.y1, A.w0, A.w1) && vec8_ok(d, A.post_w, A.pre_w, A.x, A.act) && vec8_ok(d, A.extra);
  float s0 = 0.f, s1 = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
      float a[8];
      load8(y0 + i, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) s0 = fmaf(a[j], a[j], s0);
      if (y1) {
        float b[8];
        load8(y1 + i, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) s1 = fmaf(b[j], b[j], s1);
      }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) {
      const float a = load_as_float(y0, i);
      s0 = fmaf(a, a, s0);
      if (y1) { const float b = load_as_float(y1, i); s1 = fmaf(b, b, s1); }
    }
  }
  float ss = 0.f;
  if (y1) {
    const float r0 = 1.0f / sqrtf(cta_sum(s0, s_part) / (float)d + A.eps);
    const float r1 = 1.0f / sqrtf(cta_sum(s1, s_part) / (float)d + A.eps);
    if (vec) {
      for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
        float a[8], b[8], ga[8], gb[8];
        load8(y0 + i, a); load8(y1 + i, b); load8(w0 + i, ga); load8(w1 + i, gb);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = 0.5f * (a[j] * r0 * ga[j] + b[j] * r1 * gb[j]);
          sw_row[i + j] = v;
          ss = fmaf(v, v, ss);
        }
      }
    } else {
      for (int i = threadIdx.x; i < d; i += kRowThreads) {
        const float v = 0.5f * (load_as_float(y0, i) * r0 * load_as_float(w0, i) + load_as_float(y1, i) * r1 * load_as_float(w1, i));
        sw_row[i] = v;
        ss = fmaf(v, v, ss);
      }
    }
  } else {
    if (vec) {
      for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
        float a[8];
        load8(y0 + i, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) sw_row[i + j] = a[j];
      }
    } else {
      for (int i = threadIdx.x; i < d; i += kRowThreads) sw_row[i] = load_as_float(y0, i);
    }
    ss = s0;
  }
  float rp = 1.0f;
  if (pw) rp = 1.0f / sqrtf(cta_sum(ss, s_part) / (float)d + A.eps);
  float sx = 0.f;
  // each thread touches only the elements it wrote: no barrier needed between the passes over sw_row
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
      float xv[8], g[8], e[8];
      load8(xr + i, xv);
      if (pw) load8(pw + i, g);
      if (ex) load8(ex + i, e);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = xv[j] + (pw ? sw_row[i + j] * rp * g[j] : sw_row[i + j]);
        if (ex) v += e[j];
        xv[j] = v;
        sw_row[i + j] = v;
        sx = fmaf(v, v, sx);
      }
      store8(xr + i, xv);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) {
      float v = xr[i] + (pw ? sw_row[i] * rp * load_as_float(pw, i) : sw_row[i]);
      if (ex) v += ex[i];
      xr[i] = v;
      sw_row[i] = v;
      sx = fmaf(v, v, sx);
    }
  }
  if (!nw) return;
  const float rn = 1.0f / sqrtf(cta_sum(sx, s_part) / (float)d + A.eps);
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += kRowThreads * 8) {
      float g[8], o[8];
      load8(nw + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = sw_row[i + j] * rn * g[j];
      store8(ar + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) store_from_float(ar, i, sw_row[i] * rn * load_as_float(nw, i));
  }
}

// elementwise activations: kind 0 exact gelu (erf), 1 tanh gelu, 2 silu, 3 relu^2
__device__ __forceinline__ float activate(float z, int kind) {
  if (kind == 0) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (kind == 2) return z / (1.0f + expf(-z));
  const float r = fmaxf(z, 0.f);
  return r * r;
}

template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(T* __restrict__ x, int64_t n, int kind) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) store_from_float(x, i, activate(load_as_float(x, i), kind));
}

// out[r, c] = act(in[r, c]) * in[r, ff + c]: the gated feed-forward's middle step over a fused [gate | up] product
template <typename T>
__global__ void __launch_bounds__(256) glu_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int ff, int kind) {
  griddep_launch();
  griddep_wait();
  const int64_t n = rows * ff;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / ff, c = i - r * ff;
    store_from_float(out, i, activate(load_as_float(in, r * 2 * ff + c), kind) * load_as_float(in, r * 2 * ff + ff + c));
  }
}

// xIELU in place, with the two raw parameters (p, q) read from `params`:
//   z > 0: softplus(p) z^2 + z / 2;   z <= 0: (1 / 2 + softplus(q)) (exp(z) - 1 - z) + z / 2
template <typename T>
__global__ void __launch_bounds__(256) xielu_kernel(T* __restrict__ x, int64_t n, const T* __restrict__ params) {
  griddep_launch();
  griddep_wait();
  const float ap = log1pf(expf(load_as_float(params, 0))), aq = 0.5f + log1pf(expf(load_as_float(params, 1)));
  // 16-bit rows take the fast exponential: its absolute error (about 2e-7) is far below the rounding of what is stored; fp32 rows
  // take expm1, which keeps exp(z) - 1 - z accurate for small z
  auto f = [&](float z) {
    const float neg = sizeof(T) == 2 ? __expf(fminf(z, 0.f)) - 1.0f - z : expm1f(fminf(z, 0.f)) - z;
    return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, neg, 0.5f * z);
  };
  if (vec8_ok(n, x)) {
    for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8; i < n; i += (int64_t)gridDim.x * 2048) {
      float v[8];
      load8(x + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = f(v[j]);
      store8(x + i, v);
    }
    return;
  }
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) store_from_float(x, i, f(load_as_float(x, i)));
}

// out[r, c] = g sigmoid(alpha g) (u + 1) with g = min(in[r, c], limit), u = clamp(in[r, ff + c], -limit, limit): the middle step of a
// gated feed-forward with clamped branches over a fused [gate | up] product
template <typename T>
__global__ void __launch_bounds__(256) glu_clamped_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int ff, float limit, float alpha) {
  griddep_launch();
  griddep_wait();
  auto f = [&](float g, float u) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
  };
  if (vec8_ok(ff, in, out)) {
    const int64_t n8 = rows * (ff / 8);
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n8; i += (int64_t)gridDim.x * 256) {
      const int64_t r = i / (ff / 8), c = (i - r * (ff / 8)) * 8;
      float g[8], u[8];
      load8(in + r * 2 * ff + c, g);
      load8(in + r * 2 * ff + ff + c, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = f(g[j], u[j]);
      store8(out + r * ff + c, g);
    }
    return;
  }
  const int64_t n = rows * ff;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / ff, c = i - r * ff;
    store_from_float(out, i, f(load_as_float(in, r * 2 * ff + c), load_as_float(in, r * 2 * ff + ff + c)));
  }
}

// Residual update of a block whose sublayers read one norm and are scaled per channel, fused with the norm that feeds the next
// block -- a dynamic tanh, which needs no statistics, so the kernel is elementwise:
//   x   += y0 * s0 + (y1 + y2) * s1 + extra + row_add      (fp32 stream; every term optional, a missing scale is 1)
//   cast = T(x)                                            (optional copy in the matrix-product dtype)
//   act  = T(tanh(alpha * x) * nw + nb)                    (skipped without nw)
struct ScaledResidualArgs {
  const void* y0; const void* s0; const void* y1; const void* y2; const void* s1;
  const float* extra; const void* row_add;
  float* x; void* cast;
  const void* alpha; const void* nw; const void* nb; void* act;
  int64_t rows;
  int d;
};

template <typename T, int V>
__global__ void __launch_bounds__(256) scaled_residual_kernel(ScaledResidualArgs A) {
  griddep_launch();
  griddep_wait();
  const int d = A.d, per = d / V;
  const int64_t n = A.rows * per;
  const T* y0 = reinterpret_cast<const T*>(A.y0);
  const T* y1 = reinterpret_cast<const T*>(A.y1);
  const T* y2 = reinterpret_cast<const T*>(A.y2);
  const T* s0 = reinterpret_cast<const T*>(A.s0);
  const T* s1 = reinterpret_cast<const T*>(A.s1);
  const T* ra = reinterpret_cast<const T*>(A.row_add);
  const T* nw = reinterpret_cast<const T*>(A.nw);
  const T* nb = reinterpret_cast<const T*>(A.nb);
  const bool changes = y0 || y1 || y2 || A.extra || ra;
  const float alpha = nw ? load_as_float(reinterpret_cast<const T*>(A.alpha), 0) : 0.f;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / per;
    const int c = (int)(i - r * per) * V;
    const int64_t o = r * d + c;
    float x[V], t[V], u[V], s[V];
    if constexpr (V == 8) load8(A.x + o, x);
    else x[0] = A.x[o];
    if (y0) {
      if constexpr (V == 8) { load8(y0 + o, t); if (s0) load8(s0 + c, s); }
      else { t[0] = load_as_float(y0, o); if (s0) s[0] = load_as_float(s0, c); }
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] = s0 ? fmaf(t[j], s[j], x[j]) : x[j] + t[j];
    }
    if (y1 || y2) {
#pragma unroll
      for (int j = 0; j < V; ++j) t[j] = 0.f;
      if (y1) {
        if constexpr (V == 8) load8(y1 + o, t);
        else t[0] = load_as_float(y1, o);
      }
      if (y2) {
        if constexpr (V == 8) load8(y2 + o, u);
        else u[0] = load_as_float(y2, o);
#pragma unroll
        for (int j = 0; j < V; ++j) t[j] += u[j];
      }
      if (s1) {
        if constexpr (V == 8) load8(s1 + c, s);
        else s[0] = load_as_float(s1, c);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] = s1 ? fmaf(t[j], s[j], x[j]) : x[j] + t[j];
    }
    if (A.extra) {
      if constexpr (V == 8) load8(A.extra + o, t);
      else t[0] = A.extra[o];
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] += t[j];
    }
    if (ra) {
      if constexpr (V == 8) load8(ra + c, t);
      else t[0] = load_as_float(ra, c);
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] += t[j];
    }
    if (changes) {
      if constexpr (V == 8) store8(A.x + o, x);
      else A.x[o] = x[0];
    }
    if (A.cast) {
      if constexpr (V == 8) store8(reinterpret_cast<T*>(A.cast) + o, x);
      else store_from_float(reinterpret_cast<T*>(A.cast), o, x[0]);
    }
    if (nw) {
      if constexpr (V == 8) { load8(nw + c, t); load8(nb + c, u); }
      else { t[0] = load_as_float(nw, c); u[0] = load_as_float(nb, c); }
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] = fmaf(tanhf(alpha * x[j]), t[j], u[j]);
      if constexpr (V == 8) store8(reinterpret_cast<T*>(A.act) + o, x);
      else store_from_float(reinterpret_cast<T*>(A.act), o, x[0]);
    }
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(kRowThreads) gather_rows_kernel(const T* __restrict__ src, const I* __restrict__ rows,
                                                                   T* __restrict__ dst, int d) {
  griddep_launch();
  griddep_wait();
  const int64_t r = (int64_t)rows[blockIdx.x];
  const T* sr = src + r * d;
  T* dr = dst + (int64_t)blockIdx.x * d;
  if (vec8_ok((int64_t)d * sizeof(T) / 2, sr, dr)) {   // whole 16-byte pieces
    const int n16 = d * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n16; i += kRowThreads) reinterpret_cast<uint4*>(dr)[i] = reinterpret_cast<const uint4*>(sr)[i];
  } else {
    for (int i = threadIdx.x; i < d; i += kRowThreads) dr[i] = sr[i];
  }
}

// x = relu(x)^2 in place
template <typename T>
__global__ void __launch_bounds__(256) sqrelu_kernel(T* __restrict__ x, int64_t n) {
  griddep_launch();
  griddep_wait();
  if (vec8_ok(n, x)) {
    for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8; i < n; i += (int64_t)gridDim.x * 2048) {
      float v[8];
      load8(x + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[j] = fmaxf(v[j], 0.f); v[j] *= v[j]; }
      store8(x + i, v);
    }
    return;
  }
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float v = fmaxf(load_as_float(x, i), 0.f);
    store_from_float(x, i, v * v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) scale_f32_kernel(const T* __restrict__ in, float scale, float* __restrict__ out, int64_t n) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) out[i] = load_as_float(in, i) * scale;
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_embed_pos(const int32_t* tokens, const int32_t* pos, const void* embed, const void* pos_table, float scale, float* x,
                   void* act, int64_t rows, int d, int vocab, int max_pos, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(tokens && embed && x && act && (pos || !pos_table), "b200_embed_pos: null pointer");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff && d > 0 && vocab > 0, "b200_embed_pos: bad shape");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(embed_pos_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, (cudaStream_t)stream, tokens,
                                               pos, (const T*)embed, (const T*)pos_table, scale, x, (T*)act, d, vocab, max_pos)));
  return B200_OK;
}

int b200_rms_rows(const b200_rms_rows_seg* segs, int n_segs, int64_t rows, float eps, int in_dtype, int out_dtype, b200_stream_t stream) {
  B200_CHECK_ARG(segs && (n_segs == 1 || n_segs == 2), "b200_rms_rows: one or two segments");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff, "b200_rms_rows: bad row count");
  RmsSeg s[2];
  for (int i = 0; i < 2; ++i) {
    const b200_rms_rows_seg& a = segs[i < n_segs ? i : 0];
    B200_CHECK_ARG(a.in && a.weight && a.out && a.d > 0, "b200_rms_rows: null pointer or empty row");
    s[i] = RmsSeg{a.in, a.weight, a.out, a.in_rows, a.out_rows, a.ld_in, a.ld_out, a.d, a.plus_one};
  }
  const dim3 grid((unsigned)rows, (unsigned)n_segs), block(kRowThreads);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16) B200_CUDA(launch(rms_rows_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, st, s[0], s[1], eps));
  else if (in_dtype == B200_F32 && out_dtype == B200_BF16) B200_CUDA(launch(rms_rows_kernel<float, __nv_bfloat16>, grid, block, 0, st, s[0], s[1], eps));
  else if (in_dtype == B200_F32 && out_dtype == B200_F32) B200_CUDA(launch(rms_rows_kernel<float, float>, grid, block, 0, st, s[0], s[1], eps));
  else { set_error("b200_rms_rows: unsupported dtype pair"); return B200_ERR_INVALID; }
  return B200_OK;
}

int b200_residual_norm_add(const void* y, const void* weight, float eps, float* x, void* act, int64_t rows, int d, int dtype,
                           b200_stream_t stream) {
  B200_CHECK_ARG(y && weight && x && act, "b200_residual_norm_add: null pointer");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff && d > 0, "b200_residual_norm_add: bad shape");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(residual_norm_add_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, (cudaStream_t)stream,
                                               (const T*)y, (const T*)weight, eps, x, (T*)act, d)));
  return B200_OK;
}

int b200_gather_rows(const void* src, const void* rows, int rows_is_int64, void* dst, int64_t n_rows, int d, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(src && rows && dst && n_rows > 0 && n_rows <= 0x7fffffff && d > 0, "b200_gather_rows: bad argument");
  if (rows_is_int64)
    B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(gather_rows_kernel<T, int64_t>, dim3((unsigned)n_rows), dim3(kRowThreads), 0, (cudaStream_t)stream,
                                                 (const T*)src, (const int64_t*)rows, (T*)dst, d)));
  else
    B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(gather_rows_kernel<T, int32_t>, dim3((unsigned)n_rows), dim3(kRowThreads), 0, (cudaStream_t)stream,
                                                 (const T*)src, (const int32_t*)rows, (T*)dst, d)));
  return B200_OK;
}

int b200_sqrelu(void* x, int64_t n, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(x && n > 0, "b200_sqrelu: bad argument");
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(sqrelu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (T*)x, n)));
  return B200_OK;
}

int b200_scale_f32(const void* in, float scale, float* out, int64_t n, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(in && out && n > 0, "b200_scale_f32: bad argument");
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(scale_f32_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)in, scale, out, n)));
  return B200_OK;
}

int b200_sandwich_residual(const b200_sandwich_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->y0 && a->x, "b200_sandwich_residual: null pointer");
  B200_CHECK_ARG(!a->y1 || (a->w0 && a->w1), "b200_sandwich_residual: two branches need their two norm weights");
  B200_CHECK_ARG(!a->pre_w || a->act, "b200_sandwich_residual: the next sublayer's norm needs somewhere to go");
  B200_CHECK_ARG(a->rows > 0 && a->rows <= 0x7fffffff && a->d > 0 && (size_t)a->d * sizeof(float) <= 160 * 1024, "b200_sandwich_residual: bad shape");
  const SandwichArgs A{a->y0, a->w0, a->y1, a->w1, a->post_w, a->extra, a->pre_w, a->x, a->act, a->d, a->eps};
  const size_t smem = (size_t)a->d * sizeof(float);
  B200_FLOAT_TYPES(a->dtype, T, {
    static PerDeviceOnce once;
    if (smem > 48 * 1024 && once.need()) {
      B200_CUDA(cudaFuncSetAttribute(sandwich_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      once.done();
    }
    B200_CUDA(launch(sandwich_residual_kernel<T>, dim3((unsigned)a->rows), dim3(kRowThreads), smem, (cudaStream_t)stream, A));
  });
  return B200_OK;
}

int b200_activation(void* x, int64_t n, int kind, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(x && n > 0 && kind >= 0 && kind <= 3, "b200_activation: bad argument");
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(activation_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (T*)x, n, kind)));
  return B200_OK;
}

int b200_glu(const void* in, void* out, int64_t rows, int ff, int kind, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(in && out && rows > 0 && ff > 0 && kind >= 0 && kind <= 3, "b200_glu: bad argument");
  int64_t blocks = (rows * ff + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(glu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)in, (T*)out, rows, ff, kind)));
  return B200_OK;
}

int b200_xielu(void* x, int64_t n, const void* params, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(x && params && n > 0, "b200_xielu: bad argument");
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(xielu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (T*)x, n, (const T*)params)));
  return B200_OK;
}

int b200_glu_clamped(const void* in, void* out, int64_t rows, int ff, float limit, float alpha, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(in && out && rows > 0 && ff > 0 && limit > 0.f, "b200_glu_clamped: bad argument");
  int64_t blocks = (rows * ff + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(glu_clamped_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)in, (T*)out,
                                               rows, ff, limit, alpha)));
  return B200_OK;
}

int b200_scaled_residual(const b200_scaled_residual_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->x && a->rows > 0 && a->rows <= 0x7fffffff && a->d > 0, "b200_scaled_residual: bad argument");
  B200_CHECK_ARG(!a->nw || (a->alpha && a->nb && a->act), "b200_scaled_residual: the norm needs its scalar, its offset and somewhere to go");
  const ScaledResidualArgs A{a->y0, a->s0, a->y1, a->y2, a->s1, a->extra, a->row_add, a->x, a->cast, a->alpha, a->nw, a->nb, a->act, a->rows, a->d};
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = a->d % 8 == 0 && al(a->y0) && al(a->s0) && al(a->y1) && al(a->y2) && al(a->s1) && al(a->extra) && al(a->row_add) && al(a->x) &&
                   al(a->cast) && al(a->nw) && al(a->nb) && al(a->act);
  int64_t blocks = (a->rows * (vec ? a->d / 8 : a->d) + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  B200_FLOAT_TYPES(a->dtype, T, {
    if (vec) B200_CUDA(launch(scaled_residual_kernel<T, 8>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, A));
    else B200_CUDA(launch(scaled_residual_kernel<T, 1>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, A));
  });
  return B200_OK;
}

}  // extern "C"
