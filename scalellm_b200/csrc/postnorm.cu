// postnorm.cu — kernels for decoders that normalise a sublayer's RESULT (not its input) before it
// enters an fp32 residual, and that feed every layer a learned average of all earlier layers' results.
//
//   embed     x = scale * E[tok] + B[(mul_prev * prev + mul_cur * tok) mod buckets]   (B[buckets] when a
//             sequence starts: prev < 0); the hashed pair table B is optional
//   postnorm  r = x + mult * y / sqrt(mean_g(y^2) + eps) * w     mean over the channel's group: the row is cut
//             into `groups` equal consecutive parts, each with its own root mean square
//   history   H[n - 1] = r ; x' = sum_{j < n} c[j] H[j]          (optional) the depth-weighted average
//   sumnorm   x' = (a x + y) / sqrt(mean((a x + y)^2) + eps) * w   the norm taken AFTER the sum; w one number for the
//             whole row or one per channel
//   softcap   out = cap tanh(in / cap)
//   glu       out = g sigmoid(slope g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit)
//   token gate out = gelu_tanh(a) * table[tok, col0 + c]          a per-token learned vector gates a projection
//   branches  m = 1/2 (a / rms(a) * wa + b / rms(b) * wb)  (or m = a when there is one branch and no branch weight);
//             x' = x + m / rms(m) * w ;  h = x' / rms(x') * w_next (or x' itself)   two sublayers side by side whose
//             normalised results are averaged, normalised again into the residual, and the next sublayer's input norm
//   relu^2    out = max(in, 0)^2
//
// The residual, the history, sums of squares and every transcendental are fp32; T is the activation type
// of y and of the copy of the residual that the next matrix product reads.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kRowThreads = 256;
constexpr int kSideThreads = 1024;   // the one-launch per-token term: one CTA streams two matrices, it needs the loads in flight

template <typename T>
__global__ void bigram_embed_kernel(float* __restrict__ x, T* __restrict__ h, const T* __restrict__ table,
                                    const T* __restrict__ pair_table, const int* __restrict__ tokens,
                                    const int* __restrict__ prev_tokens, int W, int vocab, int64_t buckets,
                                    int64_t mul_prev, int64_t mul_cur, float scale) {
  const int row = blockIdx.x;
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const T* src = table + (size_t)tok * W;
  const T* pair = nullptr;
  if (pair_table) {
    const int prev = prev_tokens ? prev_tokens[row] : -1;
    const int64_t r = prev < 0 ? buckets : ((int64_t)prev * mul_prev + (int64_t)tok * mul_cur) % buckets;
    pair = pair_table + (size_t)r * W;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = Num<T>::to_f(src[i]) * scale;
    if (pair) v += Num<T>::to_f(pair[i]);
    x[(size_t)row * W + i] = v;
    if (h) h[(size_t)row * W + i] = Num<T>::from_f(v);
  }
}

// The second half of a post-norm launch for one row whose sublayer result y_s [W] lies in shared memory: group
// root mean squares (warp w owns groups w, w + 8, ...), the residual add, the history and its average.
template <typename T>
__device__ __forceinline__ void postnorm_tail(float* __restrict__ x_out, T* __restrict__ h_out,
                                              const float* __restrict__ x_in, const float* y_s, float* r_s,
                                              const float* __restrict__ w, int row, int W, int groups, float mult,
                                              float eps, float* __restrict__ hist, int64_t hist_stride, int n_hist,
                                              const float* __restrict__ coef) {
  const int gs = W / groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += (int)blockDim.x / 32) {
    float ss = 0.0f;
    for (int i = lane; i < gs; i += 32) {
      const float v = y_s[g * gs + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) r_s[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  const size_t base = (size_t)row * W;
  // four channels per thread and step where a group of four lies inside one norm group and rows start on 16 bytes
  const bool vec = gs % 4 == 0 && ((reinterpret_cast<uintptr_t>(x_in) | reinterpret_cast<uintptr_t>(x_out) |
                                    reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(hist) |
                                    reinterpret_cast<uintptr_t>(h_out)) & 15) == 0 && hist_stride % 4 == 0;
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += (int)blockDim.x * 4) {
      const float4 xv = *reinterpret_cast<const float4*>(x_in + base + i);
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      const float rg = r_s[i / gs] * mult;
      float4 r;
      r.x = xv.x + rg * y_s[i] * wv.x;
      r.y = xv.y + rg * y_s[i + 1] * wv.y;
      r.z = xv.z + rg * y_s[i + 2] * wv.z;
      r.w = xv.w + rg * y_s[i + 3] * wv.w;
      if (hist) {
        *reinterpret_cast<float4*>(hist + (size_t)(n_hist - 1) * hist_stride + base + i) = r;
        const float cl = coef[n_hist - 1];
        float4 acc = make_float4(cl * r.x, cl * r.y, cl * r.z, cl * r.w);
        for (int j = n_hist - 2; j >= 0; --j) {
          const float4 hv = *reinterpret_cast<const float4*>(hist + (size_t)j * hist_stride + base + i);
          const float cj = coef[j];
          acc.x += cj * hv.x; acc.y += cj * hv.y; acc.z += cj * hv.z; acc.w += cj * hv.w;
        }
        r = acc;
      }
      *reinterpret_cast<float4*>(x_out + base + i) = r;
      if (h_out) {
        h_out[base + i] = Num<T>::from_f(r.x);
        h_out[base + i + 1] = Num<T>::from_f(r.y);
        h_out[base + i + 2] = Num<T>::from_f(r.z);
        h_out[base + i + 3] = Num<T>::from_f(r.w);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += (int)blockDim.x) {
    float r = x_in[base + i] + mult * (y_s[i] * r_s[i / gs] * w[i]);
    if (hist) {
      hist[(size_t)(n_hist - 1) * hist_stride + base + i] = r;
      float acc = coef[n_hist - 1] * r;
      for (int j = n_hist - 2; j >= 0; --j) acc += coef[j] * hist[(size_t)j * hist_stride + base + i];
      r = acc;
    }
    x_out[base + i] = r;
    if (h_out) h_out[base + i] = Num<T>::from_f(r);
  }
}

// one CTA per row; y is held in shared memory between the two passes
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
postnorm_residual_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                         const T* __restrict__ y, int64_t ldy, const float* __restrict__ w, int W, int groups,
                         float mult, float eps, float* __restrict__ hist, int64_t hist_stride, int n_hist,
                         const float* __restrict__ coef) {
  extern __shared__ __align__(16) float sm[];
  float* y_s = sm;            // [W]
  float* r_s = sm + W;        // [groups] reciprocal root mean squares
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += kRowThreads) y_s[i] = Num<T>::to_f(y[(size_t)row * ldy + i]);
  __syncthreads();
  postnorm_tail<T>(x_out, h_out, x_in, y_s, r_s, w, row, W, groups, mult, eps, hist, hist_stride, n_hist, coef);
}

// The same launch fed by the split-K partials of the matrix product that made y (fp32 [slots][rows][W], the
// contributing slots of a column group given by the product's partition): their sum is rounded to T, which is what
// the product's own reduction pass would have stored, so the reduction costs no launch of its own.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
postnorm_residual_splitk_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                                const float* __restrict__ partials, W4Plan plan, int64_t slot_stride,
                                const float* __restrict__ w, int W, int groups, float mult, float eps,
                                float* __restrict__ hist, int64_t hist_stride, int n_hist,
                                const float* __restrict__ coef) {
  extern __shared__ __align__(16) float sm[];
  float* y_s = sm;
  float* r_s = sm + W;
  const int row = blockIdx.x;
  const float* prow = partials + (size_t)row * W;
  for (int v = threadIdx.x; v < W / 8; v += kRowThreads) {
    float a[8];
    w4_sum_partials8(a, prow + v * 8, slot_stride, w4_contrib_col(plan, v * 8));
#pragma unroll
    for (int i = 0; i < 8; ++i) y_s[v * 8 + i] = rnd<T>(a[i]);
  }
  __syncthreads();
  postnorm_tail<T>(x_out, h_out, x_in, y_s, r_s, w, row, W, groups, mult, eps, hist, hist_stride, n_hist, coef);
}

// The per-token term of a layer for a few rows (decoding) in ONE launch instead of two small matrix products, the
// gate and the post-norm: a = G h (one warp per output, rounded to T like a GEMM result), gg = gelu_tanh(a) *
// table[tok, col0 + c], y = P gg (rounded to T), then the post-norm tail.  h: the row as the matrix products read it
// (T; the fp32 residual itself when T is float).  G [sd, W] and P TRANSPOSED [sd, W], row-major; rows are read 4
// elements a load where W is a multiple of 4 and the matrices start on 16-byte boundaries.
template <typename T>
__global__ void __launch_bounds__(kSideThreads)
token_side_postnorm_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                           const T* __restrict__ h, const T* __restrict__ G, const T* __restrict__ P,
                           const T* __restrict__ table, int64_t ld_table, int col0, const int* __restrict__ tokens,
                           int vocab, int sd, const float* __restrict__ w, int W, int groups, float mult, float eps,
                           float* __restrict__ hist, int64_t hist_stride, int n_hist,
                           const float* __restrict__ coef, int vec_g, int vec_p) {
  extern __shared__ __align__(16) float sm[];
  float* h_s = sm;                       // [W]  the input row
  float* y_s = h_s + W;                  // [W]
  float* g_s = y_s + W;                  // [sd rounded up to 4]
  float* r_s = g_s + ((sd + 3) / 4) * 4; // [groups]
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < W; i += kSideThreads) h_s[i] = Num<T>::to_f(h[(size_t)row * W + i]);
  __syncthreads();
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  // a warp takes up to 8 of the sd outputs at a time (c = warp + 8 k): 8 independent loads per step of the row
  constexpr int NW = kSideThreads / 32;
  for (int c0 = warp; c0 < sd; c0 += NW * 8) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    if (vec_g) {
      for (int i = lane * 4; i < W; i += 128) {
        const float4 hv = *reinterpret_cast<const float4*>(h_s + i);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = c0 + k * NW;
          if (c < sd) {
            float v[4];
            load4<T>(G + (size_t)c * W + i, v);
            acc[k] += hv.x * v[0]; acc[k] += hv.y * v[1]; acc[k] += hv.z * v[2]; acc[k] += hv.w * v[3];
          }
        }
      }
    } else {
      for (int i = lane; i < W; i += 32) {
        const float hv = h_s[i];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = c0 + k * NW;
          if (c < sd) acc[k] += hv * Num<T>::to_f(G[(size_t)c * W + i]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k * NW;
      const float sum = warp_sum(acc[k]);
      if (lane == 0 && c < sd) {
        const float a = rnd<T>(sum);
        const float gl = 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
        g_s[c] = rnd<T>(gl * Num<T>::to_f(table[(int64_t)tok * ld_table + col0 + c]));
      }
    }
  }
  __syncthreads();
  // P is given transposed, [sd, W]: neighbouring threads read neighbouring outputs' weights
  if (vec_p) {
    for (int i = threadIdx.x * 4; i < W; i += kSideThreads * 4) {
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll 8
      for (int c = 0; c < sd; ++c) {
        float v[4];
        load4<T>(P + (size_t)c * W + i, v);
        const float gc = g_s[c];
        a0 += gc * v[0]; a1 += gc * v[1]; a2 += gc * v[2]; a3 += gc * v[3];
      }
      y_s[i] = rnd<T>(a0); y_s[i + 1] = rnd<T>(a1); y_s[i + 2] = rnd<T>(a2); y_s[i + 3] = rnd<T>(a3);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += kSideThreads) {
      float acc = 0.0f;
      for (int c = 0; c < sd; ++c) acc += g_s[c] * Num<T>::to_f(P[(size_t)c * W + i]);
      y_s[i] = rnd<T>(acc);
    }
  }
  __syncthreads();
  postnorm_tail<T>(x_out, h_out, x_in, y_s, r_s, w, row, W, groups, mult, eps, hist, hist_stride, n_hist, coef);
}

// The norm after the sum for one row whose sublayer result y_s [W] lies in shared memory: s = alpha x + y replaces
// y_s, then x' = s / sqrt(mean(s^2) + eps) * w[i * w_stride] (w_stride 0: one gain for the row).
template <typename T>
__device__ __forceinline__ void sumnorm_tail(float* __restrict__ x_out, T* __restrict__ h_out,
                                             const float* __restrict__ x_in, float* y_s, float* red,
                                             const float* __restrict__ w, int w_stride, int row, int W, float alpha,
                                             float eps) {
  const size_t base = (size_t)row * W;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float s = alpha * x_in[base + i] + y_s[i];
    y_s[i] = s;
    ss += s * s;
  }
  ss = block_sum<kRowThreads>(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float v = y_s[i] * r * w[(size_t)i * w_stride];
    x_out[base + i] = v;
    if (h_out) h_out[base + i] = Num<T>::from_f(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
sumnorm_residual_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                        const T* __restrict__ y, int64_t ldy, const float* __restrict__ w, int w_stride, int W,
                        float alpha, float eps) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += kRowThreads) sm[i] = Num<T>::to_f(y[(size_t)row * ldy + i]);
  sumnorm_tail<T>(x_out, h_out, x_in, sm, red, w, w_stride, row, W, alpha, eps);   // each thread reads back its own
}

// The same launch fed by the split-K partials of the matrix product that made y (see postnorm_residual_splitk).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
sumnorm_residual_splitk_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                               const float* __restrict__ partials, W4Plan plan, int64_t slot_stride,
                               const float* __restrict__ w, int w_stride, int W, float alpha, float eps) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* prow = partials + (size_t)row * W;
  for (int v = threadIdx.x; v < W / 8; v += kRowThreads) {
    float a[8];
    w4_sum_partials8(a, prow + v * 8, slot_stride, w4_contrib_col(plan, v * 8));
#pragma unroll
    for (int i = 0; i < 8; ++i) sm[v * 8 + i] = rnd<T>(a[i]);
  }
  __syncthreads();
  sumnorm_tail<T>(x_out, h_out, x_in, sm, red, w, w_stride, row, W, alpha, eps);
}

template <typename T>
__global__ void softcap_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t total, float cap) {
  const float inv = 1.0f / cap;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = Num<T>::from_f(cap * tanhf(Num<T>::to_f(in[i]) * inv));
}

// out = x / sqrt(mean_group(x^2) + eps) * w for fp32 rows x, written as T; one CTA per row
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
group_rms_norm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, int W,
                      int groups, float eps) {
  extern __shared__ float sm[];
  float* x_s = sm;
  float* r_s = sm + W;
  const int row = blockIdx.x;
  const int gs = W / groups;
  for (int i = threadIdx.x; i < W; i += kRowThreads) x_s[i] = x[(size_t)row * W + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += kRowThreads / 32) {
    float ss = 0.0f;
    for (int i = lane; i < gs; i += 32) {
      const float v = x_s[g * gs + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) r_s[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += kRowThreads)
    out[(size_t)row * W + i] = Num<T>::from_f(x_s[i] * r_s[i / gs] * w[i]);
}

// One CTA per row: the branch results a (and b) are normalised, averaged, normalised again into the fp32 residual, and
// the new residual is handed on either as it is or under the next sublayer's input norm.  All sums in fp32.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
branch_norm_residual_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                            const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int64_t ldb,
                            const float* __restrict__ wa, const float* __restrict__ wb, const float* __restrict__ w,
                            const float* __restrict__ w_next, int W, float eps) {
  extern __shared__ __align__(16) float sm[];
  float* m_s = sm;          // [W]
  float* b_s = sm + W;      // [W]
  __shared__ float red[4][32];
  const int row = blockIdx.x;
  float sa = 0.0f, sb = 0.0f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float av = Num<T>::to_f(a[(size_t)row * lda + i]);
    m_s[i] = av;
    sa += av * av;
    if (b) {
      const float bv = Num<T>::to_f(b[(size_t)row * ldb + i]);
      b_s[i] = bv;
      sb += bv * bv;
    }
  }
  float sm2 = 0.0f;
  if (wa) {
    sa = block_sum<kRowThreads>(sa, red[0]);
    const float ra = 1.0f / sqrtf(sa / (float)W + eps);
    float rb = 0.0f;
    if (b) {
      sb = block_sum<kRowThreads>(sb, red[1]);
      rb = 1.0f / sqrtf(sb / (float)W + eps);
    }
    for (int i = threadIdx.x; i < W; i += kRowThreads) {
      float m = m_s[i] * ra * wa[i];
      if (b) m = 0.5f * (m + b_s[i] * rb * wb[i]);
      m_s[i] = m;
      sm2 += m * m;
    }
  } else {
    sm2 = sa;
  }
  sm2 = block_sum<kRowThreads>(sm2, red[2]);
  const float rm = 1.0f / sqrtf(sm2 / (float)W + eps);
  float sx = 0.0f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float r = x_in[(size_t)row * W + i] + m_s[i] * rm * w[i];
    x_out[(size_t)row * W + i] = r;
    m_s[i] = r;
    sx += r * r;
  }
  if (!h_out) return;
  if (w_next) {
    sx = block_sum<kRowThreads>(sx, red[3]);
    const float rx = 1.0f / sqrtf(sx / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += kRowThreads)
      h_out[(size_t)row * W + i] = Num<T>::from_f(m_s[i] * rx * w_next[i]);
  } else {
    for (int i = threadIdx.x; i < W; i += kRowThreads) h_out[(size_t)row * W + i] = Num<T>::from_f(m_s[i]);
  }
}

template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int n, int64_t ld_in) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const float v = fmaxf(Num<T>::to_f(in[r * ld_in + (idx - r * n)]), 0.0f);
    out[idx] = Num<T>::from_f(v * v);
  }
}

template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int n,
                                   int64_t ld_in, float limit, float slope) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    const float g = fminf(Num<T>::to_f(in[r * ld_in + c]), limit);
    const float u = fminf(fmaxf(Num<T>::to_f(in[r * ld_in + n + c]), -limit), limit);
    out[idx] = Num<T>::from_f(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
  }
}

// the same, 16 bytes of gate, of up and of the result per thread and step (16-bit types; n and ld multiples of 8)
template <typename T>
__global__ void glu_clamped_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int n,
                                       int64_t ld_in, float limit, float slope) {
  const int nv = n / 8;
  const int64_t total = rows * nv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nv;
    const int j = (int)(idx - r * nv);
    const uint4 graw = ld_v4(in + r * ld_in + j * 8), uraw = ld_v4(in + r * ld_in + n + j * 8);
    const T* gp = reinterpret_cast<const T*>(&graw);
    const T* up = reinterpret_cast<const T*>(&uraw);
    uint4 oraw;
    T* op = reinterpret_cast<T*>(&oraw);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g = fminf(Num<T>::to_f(gp[i]), limit);
      const float u = fminf(fmaxf(Num<T>::to_f(up[i]), -limit), limit);
      op[i] = Num<T>::from_f(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
    }
    st_v4(out + r * n + j * 8, oraw);
  }
}

// the clamped GLU fed by the split-K partials of the [gate | up] product (see postnorm_residual_splitk_kernel)
template <typename T>
__global__ void glu_clamped_splitk_kernel(T* __restrict__ out, const float* __restrict__ partials, W4Plan plan,
                                          int64_t slot_stride, int64_t rows, int n, float limit, float slope) {
  const int nv = n / 8;
  const int64_t total = rows * nv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nv;
    const int j = (int)(idx - r * nv);
    const float* prow = partials + r * (2 * (int64_t)n);
    float g[8], u[8];
    w4_sum_partials8(g, prow + j * 8, slot_stride, w4_contrib_col(plan, j * 8));
    w4_sum_partials8(u, prow + n + j * 8, slot_stride, w4_contrib_col(plan, n + j * 8));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gg = fminf(rnd<T>(g[i]), limit);
      const float uu = fminf(fmaxf(rnd<T>(u[i]), -limit), limit);
      out[r * n + j * 8 + i] = Num<T>::from_f(gg / (1.0f + expf(-slope * gg)) * (uu + 1.0f));
    }
  }
}

template <typename T>
__global__ void token_gated_gelu_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t ld_in,
                                        const T* __restrict__ table, int64_t ld_table, int col0,
                                        const int* __restrict__ tokens, int64_t rows, int n, int vocab) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    int tok = tokens[r];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float a = Num<T>::to_f(in[r * ld_in + c]);
    const float e = Num<T>::to_f(table[(int64_t)tok * ld_table + col0 + c]);
    const float gl = 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
    out[idx] = Num<T>::from_f(gl * e);
  }
}

#define POSTNORM_DISPATCH(dtype, ...)                                            \
  switch (dtype) {                                                               \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case B200_FP16: { using T = __half; __VA_ARGS__; break; }                    \
    case B200_FP32: { using T = float; __VA_ARGS__; break; }                     \
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);      \
  }

inline int ew_grid(int64_t total) {
  int64_t g = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_bigram_embed(float* x, void* h, const void* table, const void* pair_table, const int32_t* tokens,
                      const int32_t* prev_tokens, int64_t rows, int64_t W, int64_t vocab, int64_t buckets,
                      int64_t mul_prev, int64_t mul_cur, float scale, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x && table && tokens, "bigram_embed: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && vocab > 0 && W < (1ll << 30) && (!pair_table || buckets > 0),
                 "bigram_embed: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (bigram_embed_kernel<T><<<(unsigned)rows, 256, 0, st>>>(
                               x, static_cast<T*>(h), static_cast<const T*>(table),
                               static_cast<const T*>(pair_table), tokens, prev_tokens, (int)W, (int)vocab,
                               buckets, mul_prev, mul_cur, scale)));
  B200_LAUNCH_OK("bigram_embed_kernel");
  return B200_OK;
}

int b200_postnorm_residual(float* x_out, void* h_out, const float* x_in, const void* y, int64_t ldy,
                           const float* weight, int64_t rows, int64_t W, int64_t groups, float mult, float eps,
                           float* hist, int64_t hist_stride, int64_t n_hist, const float* coef, int dtype,
                           b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && y && weight, "postnorm_residual: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && groups > 0 && W % groups == 0 && ldy >= W && (W + groups) * 4 <= 200 * 1024,
                 "postnorm_residual: bad shape (W a multiple of groups, at most ~50K channels)");
  B200_CHECK_ARG(!hist || (n_hist > 0 && coef && hist_stride >= rows * W), "postnorm_residual: bad history");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(postnorm_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    postnorm_residual_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, static_cast<const T*>(y), ldy, weight, (int)W, (int)groups, mult,
        eps, hist, hist_stride, (int)n_hist, coef);
  });
  B200_LAUNCH_OK("postnorm_residual_kernel");
  return B200_OK;
}

static W4Plan plan_of(const int32_t* p) {
  W4Plan pl;
  pl.units = p[0]; pl.P = p[1]; pl.KT = p[2]; pl.NT = p[3]; pl.slots = p[4]; pl.nsub_log2 = p[5];
  return pl;
}

int b200_postnorm_residual_splitk(float* x_out, void* h_out, const float* x_in, const float* partials,
                                  int64_t n_slots, const int32_t* plan6, const float* weight, int64_t rows, int64_t W,
                                  int64_t groups, float mult, float eps, float* hist, int64_t hist_stride,
                                  int64_t n_hist, const float* coef, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && partials && plan6 && weight, "postnorm_residual_splitk: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && W % 8 == 0 && groups > 0 && W % groups == 0 && (W + groups) * 4 <= 200 * 1024 &&
                     n_slots == plan6[4] && n_slots <= W4_MAX_SLOTS && is_aligned(partials, 16),
                 "postnorm_residual_splitk: bad shape, or the partials are not those of the given partition");
  B200_CHECK_ARG(!hist || (n_hist > 0 && coef && hist_stride >= rows * W), "postnorm_residual_splitk: bad history");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  const W4Plan plan = plan_of(plan6);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(postnorm_residual_splitk_kernel<T>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    postnorm_residual_splitk_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, partials, plan, rows * W, weight, (int)W, (int)groups, mult, eps, hist,
        hist_stride, (int)n_hist, coef);
  });
  B200_LAUNCH_OK("postnorm_residual_splitk_kernel");
  return B200_OK;
}

int b200_sumnorm_residual(float* x_out, void* h_out, const float* x_in, const void* y, int64_t ldy,
                          const float* weight, int64_t weight_stride, int64_t rows, int64_t W, float alpha, float eps,
                          int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && y && weight, "sumnorm_residual: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && ldy >= W && W * 4 <= 200 * 1024 && (weight_stride == 0 || weight_stride == 1),
                 "sumnorm_residual: bad shape (at most ~50K channels; weight stride 0 or 1)");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)W * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(sumnorm_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    sumnorm_residual_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, static_cast<const T*>(y), ldy, weight, (int)weight_stride, (int)W, alpha,
        eps);
  });
  B200_LAUNCH_OK("sumnorm_residual_kernel");
  return B200_OK;
}

int b200_sumnorm_residual_splitk(float* x_out, void* h_out, const float* x_in, const float* partials, int64_t n_slots,
                                 const int32_t* plan6, const float* weight, int64_t weight_stride, int64_t rows,
                                 int64_t W, float alpha, float eps, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && partials && plan6 && weight, "sumnorm_residual_splitk: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && W % 8 == 0 && W * 4 <= 200 * 1024 && n_slots == plan6[4] &&
                     n_slots <= W4_MAX_SLOTS && is_aligned(partials, 16) && (weight_stride == 0 || weight_stride == 1),
                 "sumnorm_residual_splitk: bad shape, or the partials are not those of the given partition");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)W * sizeof(float);
  const W4Plan plan = plan_of(plan6);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(sumnorm_residual_splitk_kernel<T>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sumnorm_residual_splitk_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, partials, plan, rows * W, weight, (int)weight_stride, (int)W, alpha, eps);
  });
  B200_LAUNCH_OK("sumnorm_residual_splitk_kernel");
  return B200_OK;
}

int b200_softcap(void* out, const void* in, int64_t total, float cap, int dtype, b200_stream_t stream) {
  if (total == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "softcap: null pointer");
  B200_CHECK_ARG(total > 0 && cap > 0.0f, "softcap: the cap is a positive number");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (softcap_kernel<T><<<ew_grid(total), 256, 0, st>>>(static_cast<T*>(out),
                                                                              static_cast<const T*>(in), total, cap)));
  B200_LAUNCH_OK("softcap_kernel");
  return B200_OK;
}

int b200_glu_clamped_splitk(void* out, const float* partials, int64_t n_slots, const int32_t* plan6, int64_t rows,
                            int64_t n, float limit, float slope, int dtype, b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && partials && plan6, "glu_clamped_splitk: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n % 8 == 0 && n < (1ll << 30) && n_slots == plan6[4] &&
                     n_slots <= W4_MAX_SLOTS && is_aligned(partials, 16),
                 "glu_clamped_splitk: bad shape, or the partials are not those of the given partition");
  auto st = static_cast<cudaStream_t>(stream);
  const W4Plan plan = plan_of(plan6);
  POSTNORM_DISPATCH(dtype, (glu_clamped_splitk_kernel<T><<<ew_grid(rows * (n / 8)), 256, 0, st>>>(
                               static_cast<T*>(out), partials, plan, rows * 2 * n, rows, (int)n, limit, slope)));
  B200_LAUNCH_OK("glu_clamped_splitk_kernel");
  return B200_OK;
}

int b200_token_side_postnorm(float* x_out, void* h_out, const float* x_in, const void* h, const void* gate_weight,
                             const void* proj_weight, const void* table, int64_t ld_table, int64_t col0,
                             const int32_t* tokens, int64_t vocab, int64_t side_dim, const float* weight,
                             int64_t rows, int64_t W, int64_t groups, float mult, float eps, float* hist,
                             int64_t hist_stride, int64_t n_hist, const float* coef, int dtype,
                             b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && h && gate_weight && proj_weight && table && tokens && weight,
                 "token_side_postnorm: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && groups > 0 && W % groups == 0 && side_dim > 0 && vocab > 0 && col0 >= 0 &&
                     ld_table >= col0 + side_dim && (2 * W + groups + side_dim + 4) * 4 <= 200 * 1024,
                 "token_side_postnorm: bad shape");
  B200_CHECK_ARG(!hist || (n_hist > 0 && coef && hist_stride >= rows * W), "token_side_postnorm: bad history");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(2 * W + groups + side_dim + 4) * sizeof(float);
  const int esz = dtype == B200_FP32 ? 4 : 2;
  // 4 elements a load: every row of G and of the transposed P (W elements each) starts on a 4-element boundary
  const int vec_g = W % 4 == 0 && is_aligned(gate_weight, 16) && (W * esz) % (4 * esz) == 0;
  const int vec_p = W % 4 == 0 && is_aligned(proj_weight, 16);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(token_side_postnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    token_side_postnorm_kernel<T><<<(unsigned)rows, kSideThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, static_cast<const T*>(h), static_cast<const T*>(gate_weight),
        static_cast<const T*>(proj_weight), static_cast<const T*>(table), ld_table, (int)col0, tokens, (int)vocab,
        (int)side_dim, weight, (int)W, (int)groups, mult, eps, hist, hist_stride, (int)n_hist, coef, vec_g, vec_p);
  });
  B200_LAUNCH_OK("token_side_postnorm_kernel");
  return B200_OK;
}

int b200_group_rms_norm(void* out, const float* x, const float* weight, int64_t rows, int64_t W, int64_t groups,
                        float eps, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && x && weight, "group_rms_norm: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && groups > 0 && W % groups == 0 && (W + groups) * 4 <= 200 * 1024,
                 "group_rms_norm: bad shape (W a multiple of groups, at most ~50K channels)");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(group_rms_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    group_rms_norm_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(static_cast<T*>(out), x, weight, (int)W,
                                                                        (int)groups, eps);
  });
  B200_LAUNCH_OK("group_rms_norm_kernel");
  return B200_OK;
}

int b200_glu_clamped(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, float limit, float slope,
                     int dtype, b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "glu_clamped: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= 2 * n, "glu_clamped: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype != B200_FP32 && n % 8 == 0 && ld_in % 8 == 0 && is_aligned(in, 16) && is_aligned(out, 16)) {
    if (dtype == B200_BF16)
      glu_clamped_vec_kernel<__nv_bfloat16><<<ew_grid(rows * (n / 8)), 256, 0, st>>>(
          static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(in), rows, (int)n, ld_in, limit, slope);
    else
      glu_clamped_vec_kernel<__half><<<ew_grid(rows * (n / 8)), 256, 0, st>>>(
          static_cast<__half*>(out), static_cast<const __half*>(in), rows, (int)n, ld_in, limit, slope);
    B200_LAUNCH_OK("glu_clamped_vec_kernel");
    return B200_OK;
  }
  POSTNORM_DISPATCH(dtype, (glu_clamped_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                               static_cast<T*>(out), static_cast<const T*>(in), rows, (int)n, ld_in, limit, slope)));
  B200_LAUNCH_OK("glu_clamped_kernel");
  return B200_OK;
}

int b200_token_gated_gelu(void* out, const void* in, int64_t ld_in, const void* table, int64_t ld_table,
                          int64_t col0, const int32_t* tokens, int64_t rows, int64_t n, int64_t vocab, int dtype,
                          b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in && table && tokens, "token_gated_gelu: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= n && col0 >= 0 && ld_table >= col0 + n && vocab > 0,
                 "token_gated_gelu: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (token_gated_gelu_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                               static_cast<T*>(out), static_cast<const T*>(in), ld_in, static_cast<const T*>(table),
                               ld_table, (int)col0, tokens, rows, (int)n, (int)vocab)));
  B200_LAUNCH_OK("token_gated_gelu_kernel");
  return B200_OK;
}

int b200_branch_norm_residual(float* x_out, void* h_out, const float* x_in, const void* a, int64_t lda, const void* b,
                              int64_t ldb, const float* weight_a, const float* weight_b, const float* weight,
                              const float* weight_next, int64_t rows, int64_t W, float eps, int dtype,
                              b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && a && weight, "branch_norm_residual: null pointer");
  B200_CHECK_ARG(!b || (weight_a && weight_b), "branch_norm_residual: two branches take both branch weights");
  B200_CHECK_ARG(rows > 0 && W > 0 && lda >= W && (!b || ldb >= W) && 2 * W * 4 <= 200 * 1024,
                 "branch_norm_residual: bad shape (at most ~25K channels)");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)2 * W * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(branch_norm_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    branch_norm_residual_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, static_cast<const T*>(a), lda, static_cast<const T*>(b), ldb, weight_a,
        weight_b, weight, weight_next, (int)W, eps);
  });
  B200_LAUNCH_OK("branch_norm_residual_kernel");
  return B200_OK;
}

int b200_relu_squared(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, int dtype,
                      b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "relu_squared: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= n, "relu_squared: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (relu_squared_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                               static_cast<T*>(out), static_cast<const T*>(in), rows, (int)n, ld_in)));
  B200_LAUNCH_OK("relu_squared_kernel");
  return B200_OK;
}

}  // extern "C"
