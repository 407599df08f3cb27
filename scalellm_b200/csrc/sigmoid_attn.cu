// sigmoid_attn.cu — causal attention over a paged cache whose weights are sigmoids (not normalised over the keys),
// restricted to the query's own block of positions, and mixed across heads before they meet the values.
//
//     q_i, k_j <- affine maps of the row (bias added here), first `rot_dims` channels of every head turned by the
//                 position: channel t pairs with t + rot_dims / 2, angle p * inv_freq[t]
//     s_hij  = scale q_hi . k_gj ,  g = h / (H / G) ;  s <- cap tanh(s / cap)                    (cap 0: none)
//     a_hij  = sigmoid(s_hij + b_h)   for the keys j <= i with floor(j / size) = floor(i / size)  (size 0: all j <= i)
//     a'_hij = sum_h' M[h, h'] a_h'ij                                                             (M absent: a' = a)
//     o_hi   = sum_j a'_hij v_gj
// Blocks of positions are counted from position 0 of the sequence, whatever portion of it a step brings.
//
//   prepare : q rows -> fp32 [rows, H, dim]; k rows -> K cache [slots, G, dim]; v rows -> V cache [slots, G, vdim]
//             (cache entries have the activation type T)
//   attend  : CUDA cores, any type and size.  One CTA per tile of RQ consecutive rows of a sequence that share a
//             block of positions and ALL heads (the head mix needs every head's weight of a (query, key) pair);
//             keys walk in tiles of 32: scores (thread = (row, head, key)), mix (thread = (row, head, key)), weighted
//             sum (thread = value channels of a head, all rows of the tile).
// Positions, angles, scores, weights, the mix and the sums are fp32.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kPrepThreads = 128;
constexpr int kAttnThreads = 256;
constexpr int KT = 32;            // keys per tile

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
sigmoid_attn_prepare_kernel(float* __restrict__ q_out, const T* __restrict__ q_in, const T* __restrict__ k_in,
                            const T* __restrict__ v_in, int64_t ld, const float* __restrict__ q_bias,
                            const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                            T* __restrict__ k_cache, T* __restrict__ v_cache, const float* __restrict__ inv_freq,
                            const int* __restrict__ positions, const int* __restrict__ slots, int H, int G, int dim,
                            int vdim, int rot_dims) {
  const int row = blockIdx.x;
  const float pos = (float)positions[row];
  const size_t slot = (size_t)slots[row];
  const int half = rot_dims / 2;
  const int nq = H * dim, nk = G * dim, nv = G * vdim;
  // every thread owns channels of the lower half of a pair (and its partner), or an unturned channel
  for (int idx = threadIdx.x; idx < nq + nk; idx += kPrepThreads) {
    const bool is_q = idx < nq;
    const int c = is_q ? idx : idx - nq;
    const int head = c / dim, t = c - head * dim;
    if (t >= half && t < rot_dims) continue;           // written by the thread of its partner
    const T* src = (is_q ? q_in : k_in) + (size_t)row * ld;
    const float* bias = is_q ? q_bias : k_bias;
    float u = Num<T>::to_f(src[c]) + (bias ? bias[c] : 0.0f);
    if (t < half) {
      float v = Num<T>::to_f(src[c + half]) + (bias ? bias[c + half] : 0.0f);
      float sn, cs;
      sincosf(pos * inv_freq[t], &sn, &cs);
      const float ru = u * cs - v * sn, rv = v * cs + u * sn;
      if (is_q) {
        q_out[(size_t)row * nq + c] = ru;
        q_out[(size_t)row * nq + c + half] = rv;
      } else {
        k_cache[slot * nk + c] = Num<T>::from_f(ru);
        k_cache[slot * nk + c + half] = Num<T>::from_f(rv);
      }
    } else {
      if (is_q) q_out[(size_t)row * nq + c] = u;
      else k_cache[slot * nk + c] = Num<T>::from_f(u);
    }
  }
  const T* vs = v_in + (size_t)row * ld;
  for (int i = threadIdx.x; i < nv; i += kPrepThreads)
    v_cache[slot * nv + i] = Num<T>::from_f(Num<T>::to_f(vs[i]) + (v_bias ? v_bias[i] : 0.0f));
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// CTA b takes the packed rows [b * RQ, (b + 1) * RQ) of the step and works through them in runs of rows that belong
// to one sequence and lie in one block of positions: the rows of a run see the same keys up to their own position.
// With RQ = 1 (steps of single tokens) a CTA is one row.
template <typename T, int NC, int RQ>
__global__ void __launch_bounds__(kAttnThreads)
sigmoid_attn_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const T* __restrict__ k_cache,
                    const T* __restrict__ v_cache, const float* __restrict__ head_bias,
                    const float* __restrict__ head_mix, const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                    const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens,
                    const int* __restrict__ token_seq, int rows, int H, int G, int dim, int vdim, int block_size,
                    float scale, float cap, int size) {
  extern __shared__ __align__(16) float sm[];
  float* q_s = sm;                                   // [RQ][H][dim]
  float* a_s = q_s + (size_t)RQ * H * dim;           // [RQ][H][KT]  raw weights
  float* m_s = a_s + (size_t)RQ * H * KT;            // [RQ][H][KT]  mixed weights
  float* mix_s = m_s + (size_t)RQ * H * KT;          // [H][H]
  float* hb_s = mix_s + (head_mix ? H * H : 0);      // [H]
  __shared__ int slot_s[KT];
  const int R = H / G;
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  const int nout = H * vdim;
  if (head_mix)
    for (int i = threadIdx.x; i < H * H; i += kAttnThreads) mix_s[i] = head_mix[i];
  for (int i = threadIdx.x; i < H; i += kAttnThreads) hb_s[i] = head_bias ? head_bias[i] : 0.0f;

  const int slice0 = blockIdx.x * RQ;
  const int slice1 = min(slice0 + RQ, rows);
  int run0 = slice0;
  while (run0 < slice1) {
    // a run: rows of one sequence inside one block of positions
    const int seq = token_seq[run0];
    const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
    const int p0 = kv_len - q_len + (run0 - q_cu[seq]);                   // position of the run's first row
    const int j0 = size > 0 ? (p0 / size) * size : 0;                     // first visible key
    int n = min(slice1, q_cu[seq + 1]) - run0;                            // rows left of this sequence in the slice
    if (size > 0) n = min(n, j0 + size - p0);                             // ... and of this block
    const int p_last = p0 + n - 1;
    const int* table = block_tables + cu_block_lens[seq];
    __syncthreads();                                                       // the run before is done with q_s
    for (int i = threadIdx.x; i < n * H * dim; i += kAttnThreads) q_s[i] = q[(size_t)run0 * H * dim + i];
    float acc[RQ][NC];
#pragma unroll
    for (int r = 0; r < RQ; ++r)
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] = 0.0f;

    for (int t0 = j0; t0 <= p_last; t0 += KT) {
      const int nk = min(KT, p_last + 1 - t0);
      __syncthreads();                                                     // tile before consumed; q_s visible
      if (threadIdx.x < KT) {
        const int j = t0 + min((int)threadIdx.x, nk - 1);
        slot_s[threadIdx.x] = table[j / block_size] + j % block_size;
      }
      __syncthreads();
      // scores: lane = key, the warp's threads share (row, head): q is a broadcast read
      for (int p = threadIdx.x; p < n * H * KT; p += kAttnThreads) {
        const int jj = p % KT, rh = p / KT, h = rh % H, r = rh / H;
        const int j = t0 + jj;
        float a = 0.0f;
        if (jj < nk && j <= p0 + r) {
          const T* kr = k_cache + (size_t)slot_s[jj] * k_stride + (size_t)(h / R) * dim;
          const float* qh = q_s + (size_t)rh * dim;
          float d0 = 0.0f, d1 = 0.0f;
          int d = 0;
          if (dim % 4 == 0 && (reinterpret_cast<uintptr_t>(kr) % (4 * sizeof(T))) == 0) {
            for (; d < dim; d += 4) {
              float kv[4];
              load4<T>(kr + d, kv);
              d0 += qh[d] * kv[0] + qh[d + 2] * kv[2];
              d1 += qh[d + 1] * kv[1] + qh[d + 3] * kv[3];
            }
          }
          for (; d < dim; ++d) d0 += qh[d] * Num<T>::to_f(kr[d]);
          float s = (d0 + d1) * scale;
          if (cap > 0.0f) s = cap * tanhf(s / cap);
          a = sigmoidf_(s + hb_s[h]);
        }
        a_s[p] = a;
      }
      __syncthreads();
      const float* w_s = a_s;
      if (head_mix) {
        for (int p = threadIdx.x; p < n * H * KT; p += kAttnThreads) {
          const int jj = p % KT, rh = p / KT, h = rh % H, r = rh / H;
          const float* ar = a_s + (size_t)r * H * KT + jj;
          float m = 0.0f;
          for (int g = 0; g < H; ++g) m += mix_s[h * H + g] * ar[g * KT];
          m_s[p] = m;
        }
        __syncthreads();
        w_s = m_s;
      }
      // weighted sum of the values: a thread owns NC (head, channel) outputs for every row of the run
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int o = threadIdx.x + c * kAttnThreads;
        if (o < nout) {
          const int h = o / vdim, ch = o - h * vdim;
          const T* vb = v_cache + (size_t)(h / R) * vdim + ch;
          for (int jj = 0; jj < nk; ++jj) {
            const float v = Num<T>::to_f(vb[(size_t)slot_s[jj] * v_stride]);
#pragma unroll
            for (int r = 0; r < RQ; ++r)
              if (r < n) acc[r][c] += w_s[((size_t)r * H + h) * KT + jj] * v;
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int o = threadIdx.x + c * kAttnThreads;
      if (o < nout) {
#pragma unroll
        for (int r = 0; r < RQ; ++r)
          if (r < n) out[(size_t)(run0 + r) * ldo + o] = Num<T>::from_f(acc[r][c]);
      }
    }
    run0 += n;
  }
}

#define SA_DISPATCH(dtype, ...)                                                  \
  switch (dtype) {                                                               \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case B200_FP16: { using T = __half; __VA_ARGS__; break; }                    \
    case B200_FP32: { using T = float; __VA_ARGS__; break; }                     \
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);      \
  }

template <typename T, int NC, int RQ>
int launch_attn(void* out, int64_t ldo, const float* q, const void* kc, const void* vc, const float* hb,
                const float* mix, const int* q_cu, const int* kv_cu, const int* bt, const int* cbl, const int* ts,
                int64_t rows, int H, int G, int dim, int vdim, int bs, float scale, float cap, int size,
                cudaStream_t st) {
  if constexpr (NC * RQ > 32) {
    return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: %d sums per thread", NC * RQ);
  } else {
  const size_t smem = ((size_t)RQ * H * dim + 2 * (size_t)RQ * H * KT + (mix ? (size_t)H * H : 0) + H) * sizeof(float);
  if (smem > 200 * 1024) return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: %zu bytes of shared memory", smem);
  auto kern = sigmoid_attn_kernel<T, NC, RQ>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const unsigned grid = (unsigned)((rows + RQ - 1) / RQ);
  kern<<<grid, kAttnThreads, smem, st>>>(static_cast<T*>(out), ldo, q, static_cast<const T*>(kc),
                                         static_cast<const T*>(vc), hb, mix, q_cu, kv_cu, bt, cbl, ts, (int)rows, H,
                                         G, dim, vdim, bs, scale, cap, size);
  B200_LAUNCH_OK("sigmoid_attn_kernel");
  return B200_OK;
  }
}

template <typename T, int RQ>
int launch_attn_nc(int nc, void* out, int64_t ldo, const float* q, const void* kc, const void* vc, const float* hb,
                   const float* mix, const int* q_cu, const int* kv_cu, const int* bt, const int* cbl, const int* ts,
                   int64_t rows, int H, int G, int dim, int vdim, int bs, float scale, float cap, int size,
                   cudaStream_t st) {
#define SA_NC(N)                                                                                                  \
  return launch_attn<T, N, RQ>(out, ldo, q, kc, vc, hb, mix, q_cu, kv_cu, bt, cbl, ts, rows, H, G, dim, vdim, bs, \
                               scale, cap, size, st)
  if (nc <= 1) SA_NC(1);
  if (nc <= 2) SA_NC(2);
  if (nc <= 4) SA_NC(4);
  if (nc <= 8) SA_NC(8);
  if (nc <= 16) SA_NC(16);
  if (nc <= 32) SA_NC(32);
#undef SA_NC
  return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: heads x value size above %d", 32 * kAttnThreads);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_sigmoid_attn_prepare(float* q_out, const void* q_in, const void* k_in, const void* v_in, int64_t ld,
                              const float* q_bias, const float* k_bias, const float* v_bias, void* k_cache,
                              void* v_cache, const float* inv_freq, const int32_t* positions, const int32_t* slots,
                              int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t rot_dims,
                              int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q_out && q_in && k_in && v_in && k_cache && v_cache && positions && slots,
                 "sigmoid_attn_prepare: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && rot_dims >= 0 &&
                     rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq),
                 "sigmoid_attn_prepare: bad shape (heads a multiple of key/value heads, an even number of turned "
                 "channels, at most the head size)");
  auto st = static_cast<cudaStream_t>(stream);
  SA_DISPATCH(dtype, (sigmoid_attn_prepare_kernel<T><<<(unsigned)rows, kPrepThreads, 0, st>>>(
                         q_out, static_cast<const T*>(q_in), static_cast<const T*>(k_in), static_cast<const T*>(v_in),
                         ld, q_bias, k_bias, v_bias, static_cast<T*>(k_cache), static_cast<T*>(v_cache), inv_freq,
                         positions, slots, (int)H, (int)G, (int)dim, (int)vdim, (int)rot_dims)));
  B200_LAUNCH_OK("sigmoid_attn_prepare_kernel");
  return B200_OK;
}

int b200_sigmoid_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                      const float* head_bias, const float* head_mix, const int32_t* q_cu_lens,
                      const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                      const int32_t* token_seq, int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                      int64_t block_size, float scale, float cap, int64_t size, int64_t rows_per_cta, int dtype,
                      b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens &&
                     token_seq,
                 "sigmoid_attn: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && block_size > 0 &&
                     ldo >= H * vdim && size >= 0 && size < (1ll << 31),
                 "sigmoid_attn: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  const int nc = (int)((H * vdim + kAttnThreads - 1) / kAttnThreads);
  // rows per CTA: consecutive rows of a sequence share the key tiles they read; registers hold rows x nc sums
  int rq = rows_per_cta >= 8 ? 8 : (rows_per_cta >= 4 ? 4 : 1);
  while (rq > 1 && (rq * nc > 32 || (size_t)rq * H * (dim + 2 * KT) * 4 > 160 * 1024)) rq /= 2;
#define SA_RQ(N)                                                                                                     \
  SA_DISPATCH(dtype, return (launch_attn_nc<T, N>(nc, out, ldo, q, k_cache, v_cache, head_bias, head_mix, q_cu_lens, \
                                                  kv_cu_lens, block_tables, cu_block_lens, token_seq, rows, (int)H,  \
                                                  (int)G, (int)dim, (int)vdim, (int)block_size, scale, cap,          \
                                                  (int)size, st)))
  if (rq >= 8) { SA_RQ(8); }
  if (rq >= 4) { SA_RQ(4); }
  if (rq >= 2) { SA_RQ(2); }
  SA_RQ(1);
#undef SA_RQ
  return B200_OK;
}

}  // extern "C"
