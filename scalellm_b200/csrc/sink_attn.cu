// sink_attn.cu — causal softmax attention over a paged cache with unit-length queries and keys, a query
// temperature that grows with the position, a logarithmic distance bias per head and a learned sink.
//
//     q_i <- q_i / rms(q_i) * (1 + c ln(floor((i + 1) / n) + 1))      per head, no weight    (c = 0: no temperature)
//     k_j <- k_j / rms(k_j)
//     s_ij = scale q_i . k_j - r1_h ln(1 + r2_h (i - j))               j <= i                 (r1 absent: no bias)
//     p_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'))             the sink has no key and no value
//     o_i  = sum_j p_ij v_j
// Query head h reads key/value head h / (H / G).  Values may be blended with the values another layer made of the
// same token before they are cached:  v <- (1 - lam) v + lam v_other.
//
//   prepare : q rows -> fp32 [rows, H, dim]; k rows -> K cache [slots, G, dim]; v rows -> V cache [slots, G, vdim]
//             (cache entries have the activation type T)
//   attend  : CUDA cores, any type and size: one CTA per (row, key/value head, chunk of query heads); its warps are
//             query heads times a split of the keys; lane = key for the score, lane = value channels for the sum.
//   prefill : bf16 on the tensor cores (mma.sync m16n8k16): tiles of 16 consecutive tokens x 32 keys.
//   decode  : bf16 on the tensor cores, single tokens: the 16 rows of a tile are the query heads of a key/value group.
// Norms, temperature, scores, bias, softmax weights and sums are fp32.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kPrepWarps = 4;
constexpr int kMaxWarps = 16;
constexpr int kMaxVdim = 512;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
sink_attn_prepare_kernel(float* __restrict__ q_out, const T* __restrict__ q_in, const T* __restrict__ k_in,
                         const T* __restrict__ v_in, int64_t ld, const T* __restrict__ v_other, int64_t ld_other,
                         float lam, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         const int* __restrict__ positions, const int* __restrict__ slots, int H, int G, int dim,
                         int vdim, float eps, float temp_coef, int temp_every) {
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[row];
  float temp = 1.0f;
  if (temp_coef != 0.0f && temp_every > 0) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
  const size_t slot = k_in ? (size_t)slots[row] : 0;
  const int n_k = k_in ? G : 0;
  for (int u = warp; u < H + n_k; u += kPrepWarps) {
    const bool is_q = u < H;
    const T* src = is_q ? q_in + (size_t)row * ld + (size_t)u * dim : k_in + (size_t)row * ld + (size_t)(u - H) * dim;
    float ss = 0.0f;
    for (int i = lane; i < dim; i += 32) {
      const float v = Num<T>::to_f(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dim + eps);
    if (is_q) {
      float* dst = q_out + ((size_t)row * H + u) * dim;
      for (int i = lane; i < dim; i += 32) dst[i] = Num<T>::to_f(src[i]) * r * temp;
    } else {
      T* dst = k_cache + (slot * G + (u - H)) * dim;
      for (int i = lane; i < dim; i += 32) dst[i] = Num<T>::from_f(Num<T>::to_f(src[i]) * r);
    }
  }
  if (v_in) {
    const int nv = G * vdim;
    const T* vs = v_in + (size_t)row * ld;
    T* vd = v_cache + slot * nv;
    if (v_other) {
      const T* vo = v_other + (size_t)row * ld_other;
      for (int i = threadIdx.x; i < nv; i += kPrepWarps * 32)
        vd[i] = Num<T>::from_f((1.0f - lam) * Num<T>::to_f(vs[i]) + lam * Num<T>::to_f(vo[i]));
    } else {
      for (int i = threadIdx.x; i < nv; i += kPrepWarps * 32) vd[i] = vs[i];
    }
  }
}

// The end of a head's walk: its softmax denominator takes the sink, a term exp(sink) with no value.
__device__ __forceinline__ float sink_scale(float m, float l, const float* sink, int h) {
  // returns f with o_final = o * f, o accumulated relative to the running maximum m with sum l
  if (!sink) return 1.0f / l;
  const float s = sink[h];
  const float M = fmaxf(m, s);
  const float c = expf(m - M);
  return c / (l * c + expf(s - M));
}

// One CTA per (row, key/value head, chunk of RH query heads of that group); warp = (head r, key split sp).  Lane
// owns value channels lane + 32 c, c < NC.
template <typename T, int NC>
__global__ void __launch_bounds__(kMaxWarps * 32)
sink_attn_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const T* __restrict__ k_cache,
                 const T* __restrict__ v_cache, const float* __restrict__ r1, const float* __restrict__ r2,
                 const float* __restrict__ sink, const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                 const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens,
                 const int* __restrict__ token_seq, int H, int G, int dim, int vdim, int block_size, float scale,
                 int RH, int S) {
  extern __shared__ __align__(16) float sm[];
  const int n_warps = RH * S;
  float* q_s = sm;                              // [RH][dim]
  float* acc_s = q_s + RH * dim;                // [n_warps][vdim]
  float* ml_s = acc_s + n_warps * vdim;         // [n_warps][2]
  const int row = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = H / G;
  const int r = warp % RH, sp = warp / RH;
  const int h_local = blockIdx.z * RH + r;
  const bool head_ok = h_local < R;
  const int h = g * R + (head_ok ? h_local : 0);
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);            // position of this row
  const int* table = block_tables + cu_block_lens[seq];
  for (int d = threadIdx.x; d < RH * dim; d += blockDim.x) {
    const int rr = d / dim, hh = blockIdx.z * RH + rr;
    q_s[d] = hh < R ? q[((size_t)row * H + g * R + hh) * dim + (d - rr * dim)] : 0.0f;
  }
  __syncthreads();
  const float* qh = q_s + r * dim;
  const float b1 = r1 ? r1[h] : 0.0f, b2 = r1 ? r2[h] : 0.0f;
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  float m = -INFINITY, l = 0.0f;
  float acc[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) acc[c] = 0.0f;
  for (int n0 = sp * 32; n0 <= i; n0 += S * 32) {
    const int j = n0 + lane;
    const bool live = j <= i;
    // lanes past the last key point at the row's own position (always written) with weight 0
    const int jj = live ? j : i;
    const int slot = table[jj / block_size] + jj % block_size;
    float s = -INFINITY;
    if (live) {
      const T* kr = k_cache + (size_t)slot * k_stride + (size_t)g * dim;
      float d0 = 0.0f;
      for (int d = 0; d < dim; ++d) d0 += qh[d] * Num<T>::to_f(kr[d]);
      s = d0 * scale;
      if (r1) s -= b1 * logf(1.0f + b2 * (float)(i - j));
    }
    float t = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    const float nm = fmaxf(m, t);            // finite: lane 0 of a started group is live
    const float corr = expf(m - nm);
    const float p = live ? expf(s - nm) : 0.0f;
    l = l * corr + warp_sum(p);
    m = nm;
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[c] *= corr;
#pragma unroll 4
    for (int kk = 0; kk < 32; ++kk) {
      const float w = __shfl_sync(0xffffffffu, p, kk);
      const int sl = __shfl_sync(0xffffffffu, slot, kk);
      const T* vr = v_cache + (size_t)sl * v_stride + (size_t)g * vdim;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int col = lane + 32 * c;
        if (col < vdim) acc[c] += w * Num<T>::to_f(vr[col]);
      }
    }
  }
  if (lane == 0) {
    ml_s[warp * 2] = m;
    ml_s[warp * 2 + 1] = l;
  }
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int col = lane + 32 * c;
    if (col < vdim) acc_s[warp * vdim + col] = acc[c];
  }
  __syncthreads();
  if (sp != 0 || !head_ok) return;
  float M = -INFINITY;
  for (int k = 0; k < S; ++k) M = fmaxf(M, ml_s[(r + k * RH) * 2]);
  float L = 0.0f;
  float o[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) o[c] = 0.0f;
  for (int k = 0; k < S; ++k) {
    const int w = r + k * RH;
    const float f = ml_s[w * 2 + 1] > 0.0f ? expf(ml_s[w * 2] - M) : 0.0f;
    L += f * ml_s[w * 2 + 1];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) o[c] += f * acc_s[w * vdim + col];
    }
  }
  const float f = sink_scale(M, L, sink, h);
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int col = lane + 32 * c;
    if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = Num<T>::from_f(o[c] * f);
  }
}

template <typename T, int NC>
int launch_simt(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache, const float* r1,
                const float* r2, const float* sink, const int* q_cu, const int* kv_cu, const int* tables,
                const int* blk_cu, const int* token_seq, int64_t rows, int H, int G, int dim, int vdim,
                int block_size, float scale, cudaStream_t st) {
  const int R = H / G;
  const int RH = R < kMaxWarps ? R : kMaxWarps;
  int S = kMaxWarps / RH;
  if (S > 8) S = 8;
  const int chunks = (R + RH - 1) / RH;
  const int n_warps = RH * S;
  const size_t smem = ((size_t)RH * dim + (size_t)n_warps * vdim + (size_t)n_warps * 2) * sizeof(float);
  B200_CHECK_ARG(smem <= 200 * 1024, "sink_attn: head sizes %d / %d do not fit in shared memory", dim, vdim);
  auto kern = sink_attn_kernel<T, NC>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)rows, (unsigned)G, (unsigned)chunks);
  kern<<<grid, n_warps * 32, smem, st>>>(static_cast<T*>(out), ldo, q, static_cast<const T*>(k_cache),
                                         static_cast<const T*>(v_cache), r1, r2, sink, q_cu, kv_cu, tables, blk_cu,
                                         token_seq, H, G, dim, vdim, block_size, scale, RH, S);
  B200_LAUNCH_OK("sink_attn_kernel");
  return B200_OK;
}

template <typename T>
int dispatch_simt(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache, const float* r1,
                  const float* r2, const float* sink, const int* q_cu, const int* kv_cu, const int* tables,
                  const int* blk_cu, const int* token_seq, int64_t rows, int H, int G, int dim, int vdim,
                  int block_size, float scale, cudaStream_t st) {
#define SA_ARGS out, ldo, q, k_cache, v_cache, r1, r2, sink, q_cu, kv_cu, tables, blk_cu, token_seq, rows, H, G, dim, \
                vdim, block_size, scale, st
  const int nc = (vdim + 31) / 32;
  if (nc <= 1) return launch_simt<T, 1>(SA_ARGS);
  if (nc <= 2) return launch_simt<T, 2>(SA_ARGS);
  if (nc <= 4) return launch_simt<T, 4>(SA_ARGS);
  if (nc <= 8) return launch_simt<T, 8>(SA_ARGS);
  return launch_simt<T, 16>(SA_ARGS);
#undef SA_ARGS
}

// ------------------------------------------------------------------------------------------------------------
// Prompt portions in bf16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
// One CTA = 4 warps = RW query heads of one key/value group x (4 / RW) sub-tiles of 16 consecutive tokens of one
// sequence, so that all warps walk the same key tiles: 32 keys per tile, K [32][dim] and V [32][vdim] copied
// asynchronously (two buffers) through the block table.  Per warp and tile: S = Q K^T, the scale, the distance
// bias and the causal test per element, a running maximum / sum per row in fp32, and O += P V with the weights
// entering the product as two bf16 terms (p = hi + lo, 16 mantissa bits).
// ------------------------------------------------------------------------------------------------------------
constexpr int kBK = 32;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = smem_u32(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  hi = Num<__nv_bfloat16>::pack(__bfloat162float(xh), __bfloat162float(yh));
  lo = Num<__nv_bfloat16>::pack(x - __bfloat162float(xh), y - __bfloat162float(yh));
}

// dim <= 16 KS_MAX, vdim <= 16 VT_MAX, both multiples of 16; EXACT: dim = 16 KS_MAX and vdim = 16 VT_MAX, known to
// the compiler
template <int KS_MAX, int VT_MAX, bool EXACT>
__global__ void __launch_bounds__(128, EXACT ? 4 : 1)
sink_attn_prefill_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                         const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                         const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
                         const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                         const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens, int H, int G,
                         int dim_rt, int vdim_rt, int block_size, float scale, int RW, int chunks) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int dim = EXACT ? 16 * KS_MAX : dim_rt, vdim = EXACT ? 16 * VT_MAX : vdim_rt;
  const int KROW = dim + 8, VROW = vdim + 8;            // bf16 elements per staged row (16 bytes of padding)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);     // [4][16][KROW]
  __nv_bfloat16* Ks = Qs + 4 * 16 * KROW;                          // [2][kBK][KROW]
  __nv_bfloat16* Vs = Ks + 2 * kBK * KROW;                         // [2][kBK][VROW]
  const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
  const int R = H / G, TW = 4 / RW, BQ = 16 * TW;
  const int q0 = q_cu[seq], q_len = q_cu[seq + 1] - q0, kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int t0 = blockIdx.x * BQ;                       // first token of the CTA within the step's portion
  if (t0 >= q_len) return;
  const int first_pos = kv_len - q_len;
  const int hr = warp % RW, ts = warp / RW;
  const int h_local = chunk * RW + hr;
  const bool head_ok = h_local < R;
  const int h = g * R + (head_ok ? h_local : 0);
  const int KS = dim / 16, VT = vdim / 16;
  const int* table = block_tables + cu_block_lens[seq];
  {
    __nv_bfloat16* qw = Qs + warp * 16 * KROW;
    for (int e = lane; e < 16 * dim; e += 32) {
      const int rr = e / dim, d = e - rr * dim;
      const int t = t0 + ts * 16 + rr;
      const float v = (t < q_len && head_ok) ? q[((size_t)(q0 + t) * H + h) * dim + d] : 0.0f;
      qw[rr * KROW + d] = __float2bfloat16_rn(v);
    }
  }
  const int P1 = first_pos + (t0 + BQ < q_len ? t0 + BQ : q_len) - 1;   // last position of the CTA's tokens
  const int n_tiles = P1 / kBK + 1;
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  auto load_tile = [&](int idx, int buf) {
    const int key = threadIdx.x >> 2, sub = threadIdx.x & 3;
    const int j = idx * kBK + key;
    const bool ok = j <= P1;
    size_t slot = 0;
    if (ok) slot = (size_t)table[j / block_size] + j % block_size;
    const __nv_bfloat16* kr = k_cache + slot * k_stride + (size_t)g * dim;
    const __nv_bfloat16* vr = v_cache + slot * v_stride + (size_t)g * vdim;
    __nv_bfloat16* kd = Ks + ((size_t)buf * kBK + key) * KROW;
    __nv_bfloat16* vd = Vs + ((size_t)buf * kBK + key) * VROW;
    for (int c = sub; c < dim / 8; c += 4) cp_async16(kd + c * 8, kr + c * 8, ok);
    for (int c = sub; c < vdim / 8; c += 4) cp_async16(vd + c * 8, vr + c * 8, ok);
  };
  load_tile(0, 0);
  cp_async_commit();

  const int gr = lane >> 2, qc = (lane & 3) * 2;        // fragment row within 8, first column of the pair
  const int row_t[2] = {t0 + ts * 16 + gr, t0 + ts * 16 + gr + 8};
  int pos[2];
#pragma unroll
  for (int r2i = 0; r2i < 2; ++r2i) pos[r2i] = (row_t[r2i] < q_len && head_ok) ? first_pos + row_t[r2i] : -1;
  const int wpos0 = first_pos + t0 + ts * 16;           // position of the warp's first row
  const bool warp_rows_valid = head_ok && t0 + ts * 16 + 15 < q_len;
  const bool biased = r1 != nullptr;
  const float b1 = biased ? r1[h] : 0.0f, b2 = biased ? r2[h] : 0.0f;
  float mx[2] = {-INFINITY, -INFINITY}, ls[2] = {0.0f, 0.0f};
  float o[VT_MAX * 2][4];
#pragma unroll
  for (int n = 0; n < VT_MAX * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const __nv_bfloat16* qw = Qs + warp * 16 * KROW;
  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    cp_async_wait_all();
    __syncthreads();                                    // tile `it` has landed; everyone is done with tile it - 1
    if (it + 1 < n_tiles) load_tile(it + 1, buf ^ 1);
    cp_async_commit();
    const int j0 = it * kBK;
    if (j0 > wpos0 + 15) continue;                      // the whole tile lies after this warp's last row
    const bool full_tile = warp_rows_valid && j0 + kBK - 1 <= wpos0;
    const __nv_bfloat16* kt = Ks + (size_t)buf * kBK * KROW;
    const __nv_bfloat16* vt = Vs + (size_t)buf * kBK * VROW;
    float sc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS_MAX; ++ks) {
      if (ks < KS) {
        uint32_t a[4];
        ldsm_x4(a, qw + (lane & 15) * KROW + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < 2; ++np) {                // two n-tiles (16 keys) per load
          uint32_t b[4];
          ldsm_x4(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * KROW + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(sc[np * 2], a, b[0], b[1]);
          mma_bf16(sc[np * 2 + 1], a, b[2], b[3]);
        }
      }
    }
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + qc + (e & 1), i = pos[e >> 1];
        float v = sc[n][e] * scale;
        if (biased) v -= b1 * __logf(1.0f + b2 * (float)(i - j));     // (a NaN of an unseen key is replaced below)
        if (!full_tile && j > i) v = -INFINITY;
        sc[n][e] = v;
        rmax[e >> 1] = fmaxf(rmax[e >> 1], v);
      }
    float corr[2], msafe[2];
#pragma unroll
    for (int r2i = 0; r2i < 2; ++r2i) {
      rmax[r2i] = fmaxf(rmax[r2i], __shfl_xor_sync(0xffffffffu, rmax[r2i], 1));
      rmax[r2i] = fmaxf(rmax[r2i], __shfl_xor_sync(0xffffffffu, rmax[r2i], 2));
      const float nm = fmaxf(mx[r2i], rmax[r2i]);
      msafe[r2i] = nm == -INFINITY ? 0.0f : nm;
      corr[r2i] = __expf(mx[r2i] - msafe[r2i]);
      mx[r2i] = nm;
      ls[r2i] *= corr[r2i];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int n = 0; n < VT_MAX * 2; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
    uint32_t phi[2][4], plo[2][4];                      // A fragments of the two 16-key steps
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float p0 = __expf(sc[n][0] - msafe[0]), p1 = __expf(sc[n][1] - msafe[0]);
      const float p2 = __expf(sc[n][2] - msafe[1]), p3 = __expf(sc[n][3] - msafe[1]);
      ls[0] += p0 + p1;
      ls[1] += p2 + p3;
      const int kk = n >> 1, half = (n & 1) * 2;
      split_bf16(p0, p1, phi[kk][half], plo[kk][half]);
      split_bf16(p2, p3, phi[kk][half + 1], plo[kk][half + 1]);
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
      for (int vp = 0; vp < VT_MAX; vp += 2) {
        if (vp < VT) {
          const bool two = vp + 1 < VT;
          uint32_t b0[4], b1v[4] = {0u, 0u, 0u, 0u};
          const __nv_bfloat16* vrow = vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VROW + (lane >> 4) * 8;
          ldsm_x4_t(b0, vrow + vp * 16);
          if (two) ldsm_x4_t(b1v, vrow + (vp + 1) * 16);
          mma_bf16(o[vp * 2], phi[kk], b0[0], b0[1]);
          mma_bf16(o[vp * 2 + 1], phi[kk], b0[2], b0[3]);
          if (two) {
            mma_bf16(o[vp * 2 + 2], phi[kk], b1v[0], b1v[1]);
            mma_bf16(o[vp * 2 + 3], phi[kk], b1v[2], b1v[3]);
          }
          mma_bf16(o[vp * 2], plo[kk], b0[0], b0[1]);
          mma_bf16(o[vp * 2 + 1], plo[kk], b0[2], b0[3]);
          if (two) {
            mma_bf16(o[vp * 2 + 2], plo[kk], b1v[0], b1v[1]);
            mma_bf16(o[vp * 2 + 3], plo[kk], b1v[2], b1v[3]);
          }
        }
      }
  }
  cp_async_wait_all();
#pragma unroll
  for (int r2i = 0; r2i < 2; ++r2i) {
    ls[r2i] += __shfl_xor_sync(0xffffffffu, ls[r2i], 1);
    ls[r2i] += __shfl_xor_sync(0xffffffffu, ls[r2i], 2);
    if (pos[r2i] < 0) continue;
    const float f = sink_scale(mx[r2i], ls[r2i], sink, h);
    const size_t row = (size_t)q0 + row_t[r2i];
    __nv_bfloat16* dst = out + row * ldo + (size_t)h * vdim;
#pragma unroll
    for (int n = 0; n < VT_MAX * 2; ++n)
      if (n < VT * 2)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + qc) =
            Num<__nv_bfloat16>::pack(o[n][r2i * 2] * f, o[n][r2i * 2 + 1] * f);
  }
}

template <int KS_MAX, int VT_MAX, bool EXACT>
int launch_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache, const float* r1,
                   const float* r2, const float* sink, const int* q_cu, const int* kv_cu, const int* tables,
                   const int* blk_cu, int64_t n_seq, int64_t q_max, int H, int G, int dim, int vdim, int block_size,
                   float scale, cudaStream_t st) {
  const int R = H / G;
  const int RW = R >= 4 ? 4 : (R >= 2 ? 2 : 1);
  const int chunks = (R + RW - 1) / RW;
  const int BQ = 16 * (4 / RW);
  const size_t smem = ((size_t)(4 * 16 + 2 * kBK) * (dim + 8) + (size_t)2 * kBK * (vdim + 8)) * sizeof(__nv_bfloat16);
  auto kern = sink_attn_prefill_kernel<KS_MAX, VT_MAX, EXACT>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((q_max + BQ - 1) / BQ), (unsigned)n_seq, (unsigned)(G * chunks));
  kern<<<grid, 128, smem, st>>>(static_cast<__nv_bfloat16*>(out), ldo, q, static_cast<const __nv_bfloat16*>(k_cache),
                                static_cast<const __nv_bfloat16*>(v_cache), r1, r2, sink, q_cu, kv_cu, tables, blk_cu,
                                H, G, dim, vdim, block_size, scale, RW, chunks);
  B200_LAUNCH_OK("sink_attn_prefill_kernel");
  return B200_OK;
}

// ------------------------------------------------------------------------------------------------------------
// Single tokens in bf16 on the tensor cores: the 16 rows of the product are the query HEADS of one key/value group
// (all at the row's position), so one pass over the group's keys serves every head that shares them.  One CTA per
// (row, group[, chunk of 16 heads]); tiles of 64 keys are staged as above and each of the 4 warps takes 16 keys of
// every tile with accumulators of its own; the warps' running maxima, sums and weighted sums are merged through
// shared memory at the end.  A row's tiles may be shared out over n_splits such CTAs (few rows, many SMs): each then
// hands its merged sums to sink_attn_merge_kernel through a workspace; the sink joins the sum at the very end.
// ------------------------------------------------------------------------------------------------------------
constexpr int kDK = 64;
constexpr int kDS = 2;      // staged tiles: one in flight while one is consumed (a third measured slower: the walk is
                            // bound by its own latency, and shared memory bounds the CTAs per SM)

template <int KS_MAX, int VT_MAX>
__global__ void __launch_bounds__(128)
sink_attn_decode_tc_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                           const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                           const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
                           const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                           const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens,
                           const int* __restrict__ token_seq, int H, int G, int dim, int vdim, int block_size,
                           float scale, int n_splits, float* __restrict__ ws) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int KROW = dim + 8, VROW = vdim + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);     // [16][KROW]
  float* ml_s = reinterpret_cast<float*>(Qs + 16 * KROW);          // [4 warps][2: m, l][16 rows]
  float* b_s = ml_s + 4 * 2 * 16;                                  // [2: r1, r2][16 rows]
  int* slot_s = reinterpret_cast<int*>(b_s + 2 * 16);              // [2][kDK] cache rows of the keys of two tiles
  unsigned char* big = reinterpret_cast<unsigned char*>(slot_s + 2 * kDK);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(big);       // [kDS][kDK][KROW]
  __nv_bfloat16* Vs = Ks + kDS * kDK * KROW;                       // [kDS][kDK][VROW]
  float* o_s = reinterpret_cast<float*>(big);                      // after the walk: [4 warps][16][vdim]
  const int row = blockIdx.x / n_splits, split = blockIdx.x % n_splits, g = blockIdx.y, warp = threadIdx.x >> 5,
            lane = threadIdx.x & 31;
  const int R = H / G, h_base = blockIdx.z * 16;
  const int n_heads = R - h_base < 16 ? R - h_base : 16;           // valid rows of the tile
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);
  const int KS = dim / 16, VT = vdim / 16;
  const int* table = block_tables + cu_block_lens[seq];
  for (int e = threadIdx.x; e < 16 * dim; e += 128) {
    const int rr = e / dim, d = e - rr * dim;
    const float v = rr < n_heads ? q[((size_t)row * H + g * R + h_base + rr) * dim + d] : 0.0f;
    Qs[rr * KROW + d] = __float2bfloat16_rn(v);
  }
  const bool biased = r1 != nullptr;
  if (threadIdx.x < 16) {
    const bool ok = biased && threadIdx.x < n_heads;
    b_s[threadIdx.x] = ok ? r1[g * R + h_base + threadIdx.x] : 0.0f;
    b_s[16 + threadIdx.x] = ok ? r2[g * R + h_base + threadIdx.x] : 0.0f;
  }
  const int all_tiles = i / kDK + 1;
  // this CTA's share of the row's tiles (n_splits CTAs per row; an empty share hands on sums of zero)
  const int per = (all_tiles + n_splits - 1) / n_splits;
  const int tile0 = split * per;
  const int n_tiles = all_tiles - tile0 < per ? (all_tiles - tile0 > 0 ? all_tiles - tile0 : 0) : per;
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  // The cache rows of a tile's keys are looked up in the block table one tile ahead of their copy (threads 0..63, one
  // key each, into slot_s), so that the lookup's latency is off the walk's critical path; the copy itself runs with
  // consecutive lanes on consecutive 16-byte pieces of a row, a few full lines per instruction.
  auto lookup = [&](int idx) {
    if (threadIdx.x < kDK) {
      const int j = (tile0 + idx) * kDK + threadIdx.x;
      slot_s[(idx & 1) * kDK + threadIdx.x] =
          (idx < n_tiles && j <= i) ? table[j / block_size] + j % block_size : -1;
    }
  };
  const int CK = dim / 8, CV = vdim / 8;                 // 16-byte pieces per key row and value row
  auto load_tile = [&](int idx, int buf) {
    const int* sl = slot_s + (idx & 1) * kDK;
    for (int id = threadIdx.x; id < kDK * CK; id += 128) {
      const int key = id / CK, c = id - key * CK;
      const int slot = sl[key];
      cp_async16(Ks + ((size_t)buf * kDK + key) * KROW + c * 8,
                 k_cache + (size_t)(slot < 0 ? 0 : slot) * k_stride + (size_t)g * dim + c * 8, slot >= 0);
    }
    for (int id = threadIdx.x; id < kDK * CV; id += 128) {
      const int key = id / CV, c = id - key * CV;
      const int slot = sl[key];
      cp_async16(Vs + ((size_t)buf * kDK + key) * VROW + c * 8,
                 v_cache + (size_t)(slot < 0 ? 0 : slot) * v_stride + (size_t)g * vdim + c * 8, slot >= 0);
    }
  };
  lookup(0);
  lookup(1);
  __syncthreads();
  if (n_tiles > 0) load_tile(0, 0);
  cp_async_commit();
  const int gr = lane >> 2, qc = (lane & 3) * 2;
  float mx[2] = {-INFINITY, -INFINITY}, ls[2] = {0.0f, 0.0f};
  float o[VT_MAX * 2][4];
#pragma unroll
  for (int n = 0; n < VT_MAX * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  float hb1[2] = {0.0f, 0.0f}, hb2[2] = {0.0f, 0.0f};   // the bias numbers of this lane's two heads
  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    cp_async_wait_all();                                   // tile `it` has landed
    __syncthreads();                                       // and everyone is done with tile it - 1 (and Qs, b_s stand)
    if (it + 1 < n_tiles) load_tile(it + 1, buf ^ 1);
    cp_async_commit();
    lookup(it + 2);                                        // into the half of slot_s that tile `it` has left
    if (it == 0) { hb1[0] = b_s[gr]; hb1[1] = b_s[gr + 8]; hb2[0] = b_s[16 + gr]; hb2[1] = b_s[16 + gr + 8]; }
    const int j0 = (tile0 + it) * kDK + warp * 16;       // this warp's 16 keys of the tile
    if (j0 > i) continue;                                // all after the row's position
    const __nv_bfloat16* kt = Ks + ((size_t)buf * kDK + warp * 16) * KROW;
    const __nv_bfloat16* vt = Vs + ((size_t)buf * kDK + warp * 16) * VROW;
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS_MAX; ++ks) {
      if (ks < KS) {
        uint32_t a[4], b[4];
        ldsm_x4(a, Qs + (lane & 15) * KROW + ks * 16 + (lane >> 4) * 8);
        ldsm_x4(b, kt + ((lane & 7) + (lane >> 4) * 8) * KROW + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(sc[0], a, b[0], b[1]);
        mma_bf16(sc[1], a, b[2], b[3]);
      }
    }
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + qc + (e & 1);
        float v = sc[n][e] * scale;
        if (biased) v -= hb1[e >> 1] * __logf(1.0f + hb2[e >> 1] * (float)(i - j));
        if (j > i) v = -INFINITY;
        sc[n][e] = v;
        rmax[e >> 1] = fmaxf(rmax[e >> 1], v);
      }
    float corr[2], msafe[2];
#pragma unroll
    for (int r2i = 0; r2i < 2; ++r2i) {
      rmax[r2i] = fmaxf(rmax[r2i], __shfl_xor_sync(0xffffffffu, rmax[r2i], 1));
      rmax[r2i] = fmaxf(rmax[r2i], __shfl_xor_sync(0xffffffffu, rmax[r2i], 2));
      const float nm = fmaxf(mx[r2i], rmax[r2i]);
      msafe[r2i] = nm == -INFINITY ? 0.0f : nm;
      corr[r2i] = __expf(mx[r2i] - msafe[r2i]);
      mx[r2i] = nm;
      ls[r2i] *= corr[r2i];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int n = 0; n < VT_MAX * 2; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
    uint32_t phi[4], plo[4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = __expf(sc[n][0] - msafe[0]), p1 = __expf(sc[n][1] - msafe[0]);
      const float p2 = __expf(sc[n][2] - msafe[1]), p3 = __expf(sc[n][3] - msafe[1]);
      ls[0] += p0 + p1;
      ls[1] += p2 + p3;
      split_bf16(p0, p1, phi[n * 2], plo[n * 2]);
      split_bf16(p2, p3, phi[n * 2 + 1], plo[n * 2 + 1]);
    }
#pragma unroll
    for (int vt16 = 0; vt16 < VT_MAX; ++vt16) {
      if (vt16 < VT) {
        uint32_t b[4];
        ldsm_x4_t(b, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * VROW + vt16 * 16 + (lane >> 4) * 8);
        mma_bf16(o[vt16 * 2], phi, b[0], b[1]);
        mma_bf16(o[vt16 * 2 + 1], phi, b[2], b[3]);
        mma_bf16(o[vt16 * 2], plo, b[0], b[1]);
        mma_bf16(o[vt16 * 2 + 1], plo, b[2], b[3]);
      }
    }
  }
  cp_async_wait_all();
  __syncthreads();                                       // the tiles are done with: their memory takes the partial sums
#pragma unroll
  for (int r2i = 0; r2i < 2; ++r2i) {
    ls[r2i] += __shfl_xor_sync(0xffffffffu, ls[r2i], 1);
    ls[r2i] += __shfl_xor_sync(0xffffffffu, ls[r2i], 2);
    if ((lane & 3) == 0) {
      ml_s[(warp * 2 + 0) * 16 + gr + r2i * 8] = mx[r2i];
      ml_s[(warp * 2 + 1) * 16 + gr + r2i * 8] = ls[r2i];
    }
  }
#pragma unroll
  for (int n = 0; n < VT_MAX * 2; ++n)
    if (n < VT * 2) {
      float* dst = o_s + ((size_t)warp * 16) * vdim + n * 8 + qc;
      dst[(size_t)gr * vdim] = o[n][0];
      dst[(size_t)gr * vdim + 1] = o[n][1];
      dst[(size_t)(gr + 8) * vdim] = o[n][2];
      dst[(size_t)(gr + 8) * vdim + 1] = o[n][3];
    }
  __syncthreads();
  // warp w finishes heads w, w + 4, ...: lanes over the value channels
  for (int rr = warp; rr < n_heads; rr += 4) {
    float M = -INFINITY, L = 0.0f, f[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, ml_s[(w * 2 + 0) * 16 + rr]);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float lw = ml_s[(w * 2 + 1) * 16 + rr];
      f[w] = lw > 0.0f ? expf(ml_s[(w * 2 + 0) * 16 + rr] - M) : 0.0f;
      L += f[w] * lw;
    }
    const int h = g * R + h_base + rr;
    float x[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {                        // vdim <= 128: up to 4 channels per lane
      const int col = lane + 32 * c;
      x[c] = 0.0f;
      if (col < vdim) {
#pragma unroll
        for (int w = 0; w < 4; ++w) x[c] += f[w] * o_s[((size_t)w * 16 + rr) * vdim + col];
      }
    }
    if (ws) {
      // one of several CTAs of this row: hand on (M, L) and the unnormalised sum; the merge kernel ends
      float* dst = ws + (((size_t)row * H + h) * n_splits + split) * (size_t)(2 + vdim);
      if (lane == 0) { dst[0] = M; dst[1] = L; }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (lane + 32 * c < vdim) dst[2 + lane + 32 * c] = x[c];
      continue;
    }
    const float fo = sink_scale(M, L, sink, h);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = __float2bfloat16_rn(x[c] * fo);
    }
  }
}

// The end of the walk for rows whose keys were shared out over n_splits CTAs: one warp per (row, head) merges the
// shares' maxima, sums and weighted sums and lets the sink into the denominator.
__global__ void __launch_bounds__(128)
sink_attn_merge_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ ws,
                       const float* __restrict__ sink, int64_t n_pairs, int H, int vdim, int n_splits) {
  const int64_t pair = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);      // row * H + head
  const int lane = threadIdx.x & 31;
  if (pair >= n_pairs) return;
  const int64_t row = pair / H;
  const int h = (int)(pair - row * H);
  const size_t stride = (size_t)(2 + vdim);
  const float* src = ws + (size_t)pair * n_splits * stride;
  float M = -INFINITY, L = 0.0f;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, src[s * stride]);
  float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int s = 0; s < n_splits; ++s) {
    const float* p = src + s * stride;
    const float f = p[1] > 0.0f ? expf(p[0] - M) : 0.0f;
    L += f * p[1];
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (lane + 32 * c < vdim) x[c] += f * p[2 + lane + 32 * c];
  }
  const float fo = sink_scale(M, L, sink, h);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int col = lane + 32 * c;
    if (col < vdim) out[row * ldo + (size_t)h * vdim + col] = __float2bfloat16_rn(x[c] * fo);
  }
}

template <int KS_MAX, int VT_MAX>
int launch_decode_tc(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache, const float* r1,
                     const float* r2, const float* sink, const int* q_cu, const int* kv_cu, const int* tables,
                     const int* blk_cu, const int* token_seq, int64_t rows, int H, int G, int dim, int vdim,
                     int block_size, float scale, int n_splits, float* ws, cudaStream_t st) {
  const int R = H / G;
  const size_t tiles = ((size_t)kDS * kDK * (dim + 8) + (size_t)kDS * kDK * (vdim + 8)) * sizeof(__nv_bfloat16);
  const size_t sums = (size_t)4 * 16 * vdim * sizeof(float);
  const size_t smem = (size_t)16 * (dim + 8) * sizeof(__nv_bfloat16) + (4 * 2 * 16 + 2 * 16) * sizeof(float) +
                      2 * kDK * sizeof(int) + (tiles > sums ? tiles : sums);
  auto kern = sink_attn_decode_tc_kernel<KS_MAX, VT_MAX>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)(rows * n_splits), (unsigned)G, (unsigned)((R + 15) / 16));
  kern<<<grid, 128, smem, st>>>(static_cast<__nv_bfloat16*>(out), ldo, q, static_cast<const __nv_bfloat16*>(k_cache),
                                static_cast<const __nv_bfloat16*>(v_cache), r1, r2, sink, q_cu, kv_cu, tables, blk_cu,
                                token_seq, H, G, dim, vdim, block_size, scale, n_splits, n_splits > 1 ? ws : nullptr);
  B200_LAUNCH_OK("sink_attn_decode_tc_kernel");
  if (n_splits > 1) {
    const int64_t n_pairs = rows * H;
    sink_attn_merge_kernel<<<(unsigned)((n_pairs + 3) / 4), 128, 0, st>>>(static_cast<__nv_bfloat16*>(out), ldo, ws,
                                                                          sink, n_pairs, H, vdim, n_splits);
    B200_LAUNCH_OK("sink_attn_merge_kernel");
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_sink_attn_prepare(float* q_out, const void* q_in, const void* k_in, const void* v_in, int64_t ld,
                           const void* v_other, int64_t ld_other, float lam, void* k_cache, void* v_cache,
                           const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H, int64_t G,
                           int64_t dim, int64_t vdim, float eps, float temp_coef, int64_t temp_every, int dtype,
                           b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q_out && q_in && positions, "sink_attn_prepare: null pointer");
  B200_CHECK_ARG(!k_in || (v_in && k_cache && v_cache && slots), "sink_attn_prepare: keys without values or cache");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && ld >= H * dim && temp_every >= 0 &&
                     temp_every < (1ll << 31),
                 "sink_attn_prepare: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define SP_LAUNCH(T)                                                                                             \
  sink_attn_prepare_kernel<T><<<(unsigned)rows, kPrepWarps * 32, 0, st>>>(                                        \
      q_out, static_cast<const T*>(q_in), static_cast<const T*>(k_in), static_cast<const T*>(v_in), ld,            \
      static_cast<const T*>(v_other), ld_other, lam, static_cast<T*>(k_cache), static_cast<T*>(v_cache), positions, \
      slots, (int)H, (int)G, (int)dim, (int)vdim, eps, temp_coef, (int)temp_every)
  switch (dtype) {
    case B200_BF16: SP_LAUNCH(__nv_bfloat16); break;
    case B200_FP16: SP_LAUNCH(__half); break;
    case B200_FP32: SP_LAUNCH(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef SP_LAUNCH
  B200_LAUNCH_OK("sink_attn_prepare_kernel");
  return B200_OK;
}

int b200_sink_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache, const float* r1,
                   const float* r2, const float* sink, const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
                   const int32_t* block_tables, const int32_t* cu_block_lens, const int32_t* token_seq, int64_t rows,
                   int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale, int dtype,
                   b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens && token_seq,
                 "sink_attn: null pointer");
  B200_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "sink_attn: the distance bias takes both of its numbers");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && G <= 65535 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= kMaxVdim &&
                     block_size > 0 && ldo >= H * vdim,
                 "sink_attn: bad shape (value heads of at most %d channels)", kMaxVdim);
  auto st = static_cast<cudaStream_t>(stream);
#define SA_CALL(T)                                                                                                 \
  return dispatch_simt<T>(out, ldo, q, k_cache, v_cache, r1, r2, sink, q_cu_lens, kv_cu_lens, block_tables,         \
                          cu_block_lens, token_seq, rows, (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, st)
  switch (dtype) {
    case B200_BF16: SA_CALL(__nv_bfloat16);
    case B200_FP16: SA_CALL(__half);
    case B200_FP32: SA_CALL(float);
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef SA_CALL
}

int b200_sink_attn_prefill_supported(int64_t dim, int64_t vdim, int dtype) {
  return dtype == B200_BF16 && dim > 0 && vdim > 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128;
}

int b200_sink_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                           const float* r1, const float* r2, const float* sink, const int32_t* q_cu_lens,
                           const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                           int64_t n_seq, int64_t q_max, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                           int64_t block_size, float scale, int dtype, b200_stream_t stream) {
  if (n_seq == 0 || q_max == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens,
                 "sink_attn_prefill: null pointer");
  B200_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "sink_attn_prefill: the distance bias takes both of its numbers");
  B200_CHECK_ARG(b200_sink_attn_prefill_supported(dim, vdim, dtype),
                 "sink_attn_prefill: bf16 with head sizes that are multiples of 16 and at most 128");
  B200_CHECK_ARG(n_seq > 0 && n_seq <= 65535 && q_max > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 &&
                     ldo >= H * vdim && ldo % 2 == 0 && is_aligned(out, 4) && is_aligned(k_cache, 16) &&
                     is_aligned(v_cache, 16) && G * ((H / G + 3) / 4) <= 65535,
                 "sink_attn_prefill: bad shape or alignment");
  auto st = static_cast<cudaStream_t>(stream);
#define SPF_ARGS out, ldo, q, k_cache, v_cache, r1, r2, sink, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, n_seq, \
                 q_max, (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, st
  if (dim == 64 && vdim == 64) return launch_prefill<4, 4, true>(SPF_ARGS);
  if (dim == 128 && vdim == 128) return launch_prefill<8, 8, true>(SPF_ARGS);
  if (dim <= 64 && vdim <= 64) return launch_prefill<4, 4, false>(SPF_ARGS);
  return launch_prefill<8, 8, false>(SPF_ARGS);
#undef SPF_ARGS
}

int b200_sink_attn_decode_tc(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                             const float* r1, const float* r2, const float* sink, const int32_t* q_cu_lens,
                             const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                             const int32_t* token_seq, int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                             int64_t block_size, float scale, int64_t n_splits, float* workspace,
                             int64_t workspace_floats, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens && token_seq,
                 "sink_attn_decode_tc: null pointer");
  B200_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "sink_attn_decode_tc: the distance bias takes both of its numbers");
  B200_CHECK_ARG(b200_sink_attn_prefill_supported(dim, vdim, dtype),
                 "sink_attn_decode_tc: bf16 with head sizes that are multiples of 16 and at most 128");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && G <= 65535 && H % G == 0 && block_size > 0 && ldo >= H * vdim &&
                     n_splits >= 1 && rows * n_splits < (1ll << 31) && is_aligned(k_cache, 16) && is_aligned(v_cache, 16),
                 "sink_attn_decode_tc: bad shape or alignment");
  B200_CHECK_ARG(n_splits == 1 || (workspace && workspace_floats >= rows * H * n_splits * (2 + vdim)),
                 "sink_attn_decode_tc: workspace of rows * H * n_splits * (2 + vdim) floats required");
  auto st = static_cast<cudaStream_t>(stream);
#define SDT_ARGS out, ldo, q, k_cache, v_cache, r1, r2, sink, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, \
                 token_seq, rows, (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, (int)n_splits, workspace, st
  if (dim <= 64 && vdim <= 64) return launch_decode_tc<4, 4>(SDT_ARGS);
  return launch_decode_tc<8, 8>(SDT_ARGS);
#undef SDT_ARGS
}

}  // extern "C"
