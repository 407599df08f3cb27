// latent_attn.cu — attention over a paged cache of compressed key/value latents.
//
// Every cached token is one row [c (rank) | kr (rd)]: the normalised latent c, from which each
// head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), and one rotary key part kr
// shared by all heads.  With the key map folded into the query (qa_h = Uk_h^T q_h) a head's score is
//     s = (qa_h . c + qr_h . kr) * scale
// and its output is Uv_h (sum_j p_j c_j): the kernel works entirely in the latent space, as
// multi-query attention with key width rank + rd and value width rank.
//
//   latent_prepare : per token  c = rmsnorm(dkv[:rank]) * w -> cache ; kr = rope(dkv[rank:]) -> cache ;
//                    rope on the rotary part of every query head in place.  Angles pos * f_i, cos
//                    and sin in fp32; pairs are interleaved (2i, 2i+1) or, with half_pairs, (i, i + dims/2);
//                    `mult` scales cos and sin.
//   latent_attn    : causal softmax attention of packed query rows over the paged rows (with window > 0
//                    only over the last `window` keys, the row's own included); scores,
//                    weights and accumulators in fp32.  One CTA per (token, group of 8 heads), one
//                    warp per head, 32-key tiles staged once per CTA in shared memory.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kHeadsPerCta = 8;
constexpr int kTileKeys = 32;

template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ q, int64_t ldq, const T* __restrict__ dkv,
                                      int64_t ld_dkv, T* __restrict__ cache, int64_t ldc,
                                      const float* __restrict__ cw, const float* __restrict__ inv_freq,
                                      float mult, const int* __restrict__ positions,
                                      const int* __restrict__ slots, int H, int dim, int rd, int dims,
                                      int rank, float eps, int half_pairs) {
  extern __shared__ float cs[];  // [dims / 2] cos, [dims / 2] sin
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int np = dims / 2;
  const float pos = (float)positions[row];
  const T* src = dkv + (size_t)row * ld_dkv;
  T* dst = cache + (size_t)slots[row] * ldc;
  for (int i = threadIdx.x; i < np; i += blockDim.x) {
    const float a = pos * inv_freq[i];
    cs[i] = cosf(a) * mult;
    cs[np + i] = sinf(a) * mult;
  }
  float ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = Num<T>::to_f(src[i]);
    ss += v * v;
  }
  ss = block_sum<128>(ss, red);   // also orders the cos / sin table before its readers
  const float r = rsqrtf(ss / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = Num<T>::from_f(Num<T>::to_f(src[i]) * r * cw[i]);
  for (int i = threadIdx.x; i < rd - dims; i += blockDim.x) dst[rank + dims + i] = src[rank + dims + i];
  const int tasks = (H + 1) * np;
  for (int k = threadIdx.x; k < tasks; k += blockDim.x) {
    const int hh = k / np, i = k - hh * np;
    const float c = cs[i], s = cs[np + i];
    // the partner of channel i: its neighbour (pairs 2i, 2i + 1) or the channel half the turned width on (i, i + np)
    const int e0 = half_pairs ? i : 2 * i, e1 = half_pairs ? i + np : 2 * i + 1;
    if (hh < H) {
      T* p = q + (size_t)row * ldq + (size_t)hh * (dim + rd) + dim;
      const float u = Num<T>::to_f(p[e0]), v = Num<T>::to_f(p[e1]);
      p[e0] = Num<T>::from_f(u * c - v * s);
      p[e1] = Num<T>::from_f(v * c + u * s);
    } else {
      const float u = Num<T>::to_f(src[rank + e0]), v = Num<T>::to_f(src[rank + e1]);
      dst[rank + e0] = Num<T>::from_f(u * c - v * s);
      dst[rank + e1] = Num<T>::from_f(v * c + u * s);
    }
  }
}

template <typename T, typename QA, int NR>
__global__ void __launch_bounds__(kHeadsPerCta * 32)
latent_attn_kernel(T* __restrict__ out, int64_t out_hs, int64_t out_ts, const QA* __restrict__ qa,
                   int64_t qa_hs, int64_t qa_ts, const T* __restrict__ q, int64_t ldq,
                   const T* __restrict__ cache, int64_t ldc, const int* __restrict__ q_cu,
                   const int* __restrict__ kv_cu, const int* __restrict__ tables,
                   const int* __restrict__ blk_cu, const int* __restrict__ token_seq, int H, int dim,
                   int rd, int rank, int block_size, float scale, int window) {
  extern __shared__ float sm[];
  const int Dk = rank + rd, ldk = Dk + 1;
  float* qs = sm;                           // [kHeadsPerCta][Dk]
  float* Ks = sm + kHeadsPerCta * Dk;       // [kTileKeys][ldk]
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * kHeadsPerCta + warp;
  const int seq = token_seq[row];
  const int q_len = q_cu[seq + 1] - q_cu[seq], kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int pos = kv_len - q_len + (row - q_cu[seq]);   // last visible key
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;   // first visible key
  const int* table = tables + blk_cu[seq];
  if (h < H) {
    const QA* a = qa + (size_t)h * qa_hs + (size_t)row * qa_ts;
    for (int d = lane; d < rank; d += 32) qs[warp * Dk + d] = Num<QA>::to_f(a[d]);
    const T* r = q + (size_t)row * ldq + (size_t)h * (dim + rd) + dim;
    for (int d = lane; d < rd; d += 32) qs[warp * Dk + rank + d] = Num<T>::to_f(r[d]);
  }
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  for (int j0 = lo / kTileKeys * kTileKeys; j0 <= pos; j0 += kTileKeys) {
    __syncthreads();   // previous tile fully consumed (and qs written, first time round)
    for (int jj = warp; jj < kTileKeys; jj += kHeadsPerCta) {
      const int key = j0 + jj;
      float* dstk = Ks + jj * ldk;
      if (key <= pos && key >= lo) {
        const T* srck = cache + ((size_t)table[key / block_size] + key % block_size) * ldc;
        for (int d = lane; d < Dk; d += 32) dstk[d] = Num<T>::to_f(srck[d]);
      } else {
        for (int d = lane; d < Dk; d += 32) dstk[d] = 0.0f;
      }
    }
    __syncthreads();
    if (h < H) {
      const float* qh = qs + warp * Dk;
      const float* kj = Ks + lane * ldk;
      float s = 0.0f;
      for (int d = 0; d < Dk; ++d) s += qh[d] * kj[d];
      s = (j0 + lane <= pos && j0 + lane >= lo) ? s * scale : -INFINITY;
      float mx = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m, mx);
      const float p = expf(s - m_new);
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NR; ++i) acc[i] *= corr;
      for (int jj = 0; jj < kTileKeys; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const float* kr = Ks + jj * ldk;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = lane + 32 * i;
          if (r < rank) acc[i] += pj * kr[r];
        }
      }
    }
  }
  if (h < H) {
    const float inv = 1.0f / l;
    T* o = out + (size_t)h * out_hs + (size_t)row * out_ts;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = lane + 32 * i;
      if (r < rank) o[r] = Num<T>::from_f(acc[i] * inv);
    }
  }
}

template <typename T, typename QA, int NR>
int launch_latent_attn(void* out, int64_t out_hs, int64_t out_ts, const void* qa, int64_t qa_hs,
                       int64_t qa_ts, const void* q, int64_t ldq, const void* cache, int64_t ldc,
                       const int* q_cu, const int* kv_cu, const int* tables, const int* blk_cu,
                       const int* token_seq, int64_t rows, int H, int dim, int rd, int rank,
                       int block_size, float scale, int window, cudaStream_t st) {
  const int Dk = rank + rd;
  const size_t smem = ((size_t)kHeadsPerCta * Dk + (size_t)kTileKeys * (Dk + 1)) * sizeof(float);
  B200_CHECK_ARG(smem <= 200 * 1024, "latent_attn: rank + rot_dim = %d does not fit in shared memory", Dk);
  auto kern = latent_attn_kernel<T, QA, NR>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)rows, (unsigned)((H + kHeadsPerCta - 1) / kHeadsPerCta));
  kern<<<grid, kHeadsPerCta * 32, smem, st>>>(static_cast<T*>(out), out_hs, out_ts,
                                              static_cast<const QA*>(qa), qa_hs, qa_ts,
                                              static_cast<const T*>(q), ldq, static_cast<const T*>(cache),
                                              ldc, q_cu, kv_cu, tables, blk_cu, token_seq, H, dim, rd, rank,
                                              block_size, scale, window);
  B200_LAUNCH_OK("latent_attn_kernel");
  return B200_OK;
}

template <typename T, typename QA>
int dispatch_nr(int rank, void* out, int64_t out_hs, int64_t out_ts, const void* qa, int64_t qa_hs,
                int64_t qa_ts, const void* q, int64_t ldq, const void* cache, int64_t ldc, const int* q_cu,
                const int* kv_cu, const int* tables, const int* blk_cu, const int* token_seq, int64_t rows,
                int H, int dim, int rd, int block_size, float scale, int window, cudaStream_t st) {
#define LA_ARGS out, out_hs, out_ts, qa, qa_hs, qa_ts, q, ldq, cache, ldc, q_cu, kv_cu, tables, blk_cu, \
                token_seq, rows, H, dim, rd, rank, block_size, scale, window, st
  const int nr = (rank + 31) / 32;
  if (nr <= 2) return launch_latent_attn<T, QA, 2>(LA_ARGS);
  if (nr <= 4) return launch_latent_attn<T, QA, 4>(LA_ARGS);
  if (nr <= 8) return launch_latent_attn<T, QA, 8>(LA_ARGS);
  if (nr <= 16) return launch_latent_attn<T, QA, 16>(LA_ARGS);
  if (nr <= 32) return launch_latent_attn<T, QA, 32>(LA_ARGS);
#undef LA_ARGS
  return set_error(B200_ERR_UNSUPPORTED, "latent_attn: latent rank %d > 1024", rank);
}


// ---------------------------------------------------------------------------------------------
// Tensor-core form (bf16 cache): one CTA per (token, group of 16 heads, split of the keys), 4 warps.
// Per 32-key tile: warp w forms S for keys 8w..8w+7 (mma.m16n8k16 over the key width, Q and the
// tile in shared memory, fragments by ldmatrix) and does the online softmax of those 8 keys in fp32
// (the warps' row maxima and sums meet in shared memory); the weights P go to shared memory and every
// warp multiplies them by its own quarter of the latent columns (the tile read transposed by
// ldmatrix.trans).  P enters the tensor core as two bf16 terms, hi + lo: 16 bits of mantissa.  With more than one split each CTA
// writes an unnormalised partial (fp32) with its running maximum and sum; latent_combine merges them.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaRows = 16;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
  hi = Num<__nv_bfloat16>::pack(__bfloat162float(hx), __bfloat162float(hy));
  lo = Num<__nv_bfloat16>::pack(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

template <typename QA, int NTV>
__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(__nv_bfloat16* __restrict__ out, int64_t out_hs, int64_t out_ts,
                       float* __restrict__ o_part, float* __restrict__ ml_part, int n_splits,
                       const QA* __restrict__ qa, int64_t qa_hs, int64_t qa_ts,
                       const __nv_bfloat16* __restrict__ q, int64_t ldq,
                       const __nv_bfloat16* __restrict__ cache, int64_t ldc, const int* __restrict__ q_cu,
                       const int* __restrict__ kv_cu, const int* __restrict__ tables,
                       const int* __restrict__ blk_cu, const int* __restrict__ token_seq, int rows, int H,
                       int dim, int rd, int rank, int block_size, float scale, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Dk = rank + rd, DkP = (Dk + 31) / 32 * 32, ld = DkP + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][ld]
  __nv_bfloat16* Kbuf = Qs + kMmaRows * ld;                         // 2 x [32][ld], + 16 slack
  constexpr int ldp = 40;                                                   // 32 keys + 8 of padding
  __nv_bfloat16* Ph = Kbuf + 2 * kTileKeys * ld + 16;                       // [16][ldp] weights, high part
  __nv_bfloat16* Pl = Ph + kMmaRows * ldp;                                  // [16][ldp] weights, low part
  float* Wmax = reinterpret_cast<float*>(Pl + kMmaRows * ldp);              // [16][4] row maximum per warp
  float* Wsum = Wmax + kMmaRows * 4;                                        // [16][4] row sum per warp
  const int row = blockIdx.x, hg = blockIdx.y, z = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int seq = token_seq[row];
  const int q_len = q_cu[seq + 1] - q_cu[seq], kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int pos = kv_len - q_len + (row - q_cu[seq]);
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;   // first visible key
  const int* table = tables + blk_cu[seq];
  // stage Q: row r of the tile is head hg * 16 + r of this token: [folded query (rank) | rotary part (rd) | 0]
  for (int r = warp; r < kMmaRows; r += 4) {
    const int h = hg * kMmaRows + r;
    const bool live = h < H;
    const QA* a = qa + (size_t)(live ? h : 0) * qa_hs + (size_t)row * qa_ts;
    const __nv_bfloat16* qr = q + (size_t)row * ldq + (size_t)(live ? h : 0) * (dim + rd) + dim - rank;
#pragma unroll 4
    for (int d = lane; d < ld; d += 32) {
      float v = 0.0f;
      if (live && d < rank) v = Num<QA>::to_f(a[d]);
      else if (live && d < Dk) v = __bfloat162float(qr[d]);
      Qs[r * ld + d] = __float2bfloat16_rn(v);
    }
  }
  const int tile_lo = lo / kTileKeys, tiles_total = pos / kTileKeys + 1;        // tiles tile_lo .. tiles_total - 1
  const int tps = (tiles_total - tile_lo + n_splits - 1) / n_splits;
  const int tile0 = tile_lo + z * tps, tile1 = min(tiles_total, tile0 + tps);
  float acc[NTV][4];
#pragma unroll
  for (int i = 0; i < NTV; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // rows g and g + 8
  const int chunks = ld / 8;                                     // 16-byte chunks of a staged row
  const int rank8 = (rank + 7) / 8 * 8;
  // the tile's rows arrive by 16-byte asynchronous copies into one of two buffers: tile i + 1 is in flight
  // while tile i is used.  Rows beyond the last visible key and the padding chunks are zero-filled (size 0).
  const uint32_t lane_dst = lane * 16;                       // byte offset of this lane's first chunk in a row
  auto fetch = [&](int tile, __nv_bfloat16* Kd) {
    // lanes 0..7 resolve this warp's eight keys (row warp + 4 i of the tile) through the block table, once
    const int my_key = tile * kTileKeys + warp + 4 * (lane & 7);
    long long my_off = -1;
    if (my_key <= pos) my_off = ((long long)table[my_key / block_size] + my_key % block_size) * ldc;
    const uint32_t kd = smem_u32(Kd) + lane_dst;
#pragma unroll
    for (int i = 0; i < kTileKeys / 4; ++i) {
      const long long off = __shfl_sync(0xffffffffu, my_off, i);
      const __nv_bfloat16* src = cache + (off >= 0 ? off : 0) + lane * 8;
      const uint32_t dst = kd + (uint32_t)(warp + 4 * i) * (uint32_t)(ld * 2);
      for (int c = lane, it = 0; c < chunks; c += 32, ++it) {
        const int nbytes = (off >= 0 && c * 8 < Dk) ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + it * 512), "l"(nbytes ? src + it * 256 : cache), "r"(nbytes) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (tile0 < tile1) fetch(tile0, Kbuf);
  for (int tile = tile0; tile < tile1; ++tile) {
    const int j0 = tile * kTileKeys;
    __nv_bfloat16* Ks = Kbuf + ((tile - tile0) & 1) * kTileKeys * ld;
    if (tile + 1 < tile1) {
      fetch(tile + 1, Kbuf + ((tile + 1 - tile0) & 1) * kTileKeys * ld);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // S[16 x 8] of this warp's keys
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // two chains
    {
      const __nv_bfloat16* qp = Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
      const __nv_bfloat16* kp = Ks + (warp * 8 + (lane & 7)) * ld + (lane >> 3) * 8;
#pragma unroll 2
      for (int k0 = 0; k0 < DkP; k0 += 32) {
        uint32_t a[4], a2[4], b[4];
        ldsm_x4(a, qp + k0);
        ldsm_x4(a2, qp + k0 + 16);
        ldsm_x4(b, kp + k0);
        mma_bf16(s, a, b[0], b[1]);
        mma_bf16(sb, a2, b[2], b[3]);
      }
      s[0] += sb[0]; s[1] += sb[1]; s[2] += sb[2]; s[3] += sb[3];
    }
    // online softmax, each warp for its own 8 keys: local row maxima meet in shared memory, the weights go
    // back there as two bf16 terms (hi + lo) and every warp reads them as the A operand of P V
    float sv[4];
    {
      const int key = j0 + warp * 8 + 2 * t;
      const bool v0 = key <= pos && key >= lo, v1 = key + 1 <= pos && key + 1 >= lo;
      const bool r0 = hg * kMmaRows + g < H, r1 = hg * kMmaRows + g + 8 < H;
      sv[0] = (v0 && r0) ? s[0] * scale : -INFINITY;
      sv[1] = (v1 && r0) ? s[1] * scale : -INFINITY;
      sv[2] = (v0 && r1) ? s[2] * scale : -INFINITY;
      sv[3] = (v1 && r1) ? s[3] * scale : -INFINITY;
    }
    float mx0 = fmaxf(sv[0], sv[1]), mx1 = fmaxf(sv[2], sv[3]);
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    if (t == 0) { Wmax[g * 4 + warp] = mx0; Wmax[(g + 8) * 4 + warp] = mx1; }
    __syncthreads();
    const float4 wm0 = *reinterpret_cast<const float4*>(Wmax + g * 4);
    const float4 wm1 = *reinterpret_cast<const float4*>(Wmax + (g + 8) * 4);
    const float n0 = fmaxf(m0, fmaxf(fmaxf(wm0.x, wm0.y), fmaxf(wm0.z, wm0.w)));
    const float n1 = fmaxf(m1, fmaxf(fmaxf(wm1.x, wm1.y), fmaxf(wm1.z, wm1.w)));
    const bool e0 = n0 == -INFINITY, e1 = n1 == -INFINITY;       // nothing visible yet (padding rows)
    const float pa = e0 ? 0.0f : expf(sv[0] - n0), pb = e0 ? 0.0f : expf(sv[1] - n0);
    const float pc = e1 ? 0.0f : expf(sv[2] - n1), pd = e1 ? 0.0f : expf(sv[3] - n1);
    float sum0 = pa + pb, sum1 = pc + pd;
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, o);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, o);
    }
    if (t == 0) { Wsum[g * 4 + warp] = sum0; Wsum[(g + 8) * 4 + warp] = sum1; }
    {
      uint32_t hi, lo;
      split_bf16(pa, pb, hi, lo);
      *reinterpret_cast<uint32_t*>(Ph + g * ldp + warp * 8 + 2 * t) = hi;
      *reinterpret_cast<uint32_t*>(Pl + g * ldp + warp * 8 + 2 * t) = lo;
      split_bf16(pc, pd, hi, lo);
      *reinterpret_cast<uint32_t*>(Ph + (g + 8) * ldp + warp * 8 + 2 * t) = hi;
      *reinterpret_cast<uint32_t*>(Pl + (g + 8) * ldp + warp * 8 + 2 * t) = lo;
    }
    __syncthreads();
    const float c0 = e0 ? 1.0f : expf(m0 - n0), c1 = e1 ? 1.0f : expf(m1 - n1);
    {
      const float4 ws0 = *reinterpret_cast<const float4*>(Wsum + g * 4);
      const float4 ws1 = *reinterpret_cast<const float4*>(Wsum + (g + 8) * 4);
      l0 = l0 * c0 + ((ws0.x + ws0.y) + (ws0.z + ws0.w));
      l1 = l1 * c1 + ((ws1.x + ws1.y) + (ws1.z + ws1.w));
      m0 = n0; m1 = n1;
    }
    uint32_t ph[2][4], pl[2][4];
    {
      const int prow = (lane & 7) + ((lane >> 3) & 1) * 8, pcol = (lane >> 4) * 8;
      ldsm_x4(ph[0], Ph + prow * ldp + pcol);
      ldsm_x4(ph[1], Ph + prow * ldp + 16 + pcol);
      ldsm_x4(pl[0], Pl + prow * ldp + pcol);
      ldsm_x4(pl[1], Pl + prow * ldp + 16 + pcol);
    }
#pragma unroll
    for (int nt = 0; nt < NTV; nt += 2) {
      const int col0 = (warp * NTV + nt) * 8;
      if (col0 >= rank8) break;
      acc[nt][0] *= c0; acc[nt][1] *= c0; acc[nt][2] *= c1; acc[nt][3] *= c1;
      if (nt + 1 < NTV) { acc[nt + 1][0] *= c0; acc[nt + 1][1] *= c0; acc[nt + 1][2] *= c1; acc[nt + 1][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t b[4];
        ldsm_x4_t(b, Ks + (16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + col0 + (lane >> 4) * 8);
        mma_bf16(acc[nt], ph[kk], b[0], b[1]);
        mma_bf16(acc[nt], pl[kk], b[0], b[1]);
        if (nt + 1 < NTV) {
          mma_bf16(acc[nt + 1], ph[kk], b[2], b[3]);
          mma_bf16(acc[nt + 1], pl[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();   // this tile's buffer and the score tile are free again
  }
  // epilogue
  const int h0 = hg * kMmaRows + g, h1 = h0 + 8;
  if (n_splits == 1) {
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt) {
      const int col = (warp * NTV + nt) * 8 + 2 * t;
      if (h0 < H) {
        __nv_bfloat16* o = out + (size_t)h0 * out_hs + (size_t)row * out_ts;
        if (col < rank) o[col] = __float2bfloat16_rn(acc[nt][0] * i0);
        if (col + 1 < rank) o[col + 1] = __float2bfloat16_rn(acc[nt][1] * i0);
      }
      if (h1 < H) {
        __nv_bfloat16* o = out + (size_t)h1 * out_hs + (size_t)row * out_ts;
        if (col < rank) o[col] = __float2bfloat16_rn(acc[nt][2] * i1);
        if (col + 1 < rank) o[col + 1] = __float2bfloat16_rn(acc[nt][3] * i1);
      }
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt) {
      const int col = (warp * NTV + nt) * 8 + 2 * t;
      if (h0 < H) {
        float* o = o_part + (((size_t)z * rows + row) * H + h0) * rank;
        if (col < rank) o[col] = acc[nt][0];
        if (col + 1 < rank) o[col + 1] = acc[nt][1];
      }
      if (h1 < H) {
        float* o = o_part + (((size_t)z * rows + row) * H + h1) * rank;
        if (col < rank) o[col] = acc[nt][2];
        if (col + 1 < rank) o[col + 1] = acc[nt][3];
      }
    }
    if (warp == 0 && t == 0) {
      if (h0 < H) {
        float* ml = ml_part + (((size_t)z * rows + row) * H + h0) * 2;
        ml[0] = m0; ml[1] = l0;
      }
      if (h1 < H) {
        float* ml = ml_part + (((size_t)z * rows + row) * H + h1) * 2;
        ml[0] = m1; ml[1] = l1;
      }
    }
  }
}

__global__ void latent_combine_kernel(__nv_bfloat16* __restrict__ out, int64_t out_hs, int64_t out_ts,
                                      const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                      int n_splits, int rows, int H, int rank) {
  const int row = blockIdx.x, h = blockIdx.y;
  float M = -INFINITY;
  for (int z = 0; z < n_splits; ++z) M = fmaxf(M, ml_part[(((size_t)z * rows + row) * H + h) * 2]);
  float L = 0.0f;
  for (int z = 0; z < n_splits; ++z) {
    const float* ml = ml_part + (((size_t)z * rows + row) * H + h) * 2;
    if (ml[0] != -INFINITY) L += expf(ml[0] - M) * ml[1];
  }
  const float inv = 1.0f / L;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float a = 0.0f;
    for (int z = 0; z < n_splits; ++z) {
      const size_t base = ((size_t)z * rows + row) * H + h;
      const float mz = ml_part[base * 2];
      if (mz != -INFINITY) a += expf(mz - M) * o_part[base * rank + c];
    }
    out[(size_t)h * out_hs + (size_t)row * out_ts + c] = __float2bfloat16_rn(a * inv);
  }
}

template <typename QA, int NTV>
int launch_latent_mma(void* out, int64_t out_hs, int64_t out_ts, float* o_part, float* ml_part, int n_splits,
                      const void* qa, int64_t qa_hs, int64_t qa_ts, const void* q, int64_t ldq,
                      const void* cache, int64_t ldc, const int* q_cu, const int* kv_cu, const int* tables,
                      const int* blk_cu, const int* token_seq, int64_t rows, int H, int dim, int rd, int rank,
                      int block_size, float scale, int window, cudaStream_t st) {
  const int DkP = (rank + rd + 31) / 32 * 32, ld = DkP + 8;
  const size_t smem = ((size_t)(kMmaRows + 2 * kTileKeys) * ld + 16 + 2 * kMmaRows * 40) * sizeof(__nv_bfloat16) +
                      2 * kMmaRows * 4 * sizeof(float);
  B200_CHECK_ARG(smem <= 220 * 1024, "latent_attn: rank + rot_dim = %d does not fit in shared memory", rank + rd);
  auto kern = latent_attn_mma_kernel<QA, NTV>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)rows, (unsigned)((H + kMmaRows - 1) / kMmaRows), (unsigned)n_splits);
  kern<<<grid, 128, smem, st>>>(static_cast<__nv_bfloat16*>(out), out_hs, out_ts, o_part, ml_part, n_splits,
                                static_cast<const QA*>(qa), qa_hs, qa_ts, static_cast<const __nv_bfloat16*>(q), ldq,
                                static_cast<const __nv_bfloat16*>(cache), ldc, q_cu, kv_cu, tables, blk_cu,
                                token_seq, (int)rows, H, dim, rd, rank, block_size, scale, window);
  B200_LAUNCH_OK("latent_attn_mma_kernel");
  if (n_splits > 1) {
    latent_combine_kernel<<<dim3((unsigned)rows, (unsigned)H), 128, 0, st>>>(
        static_cast<__nv_bfloat16*>(out), out_hs, out_ts, o_part, ml_part, n_splits, (int)rows, H, rank);
    B200_LAUNCH_OK("latent_combine_kernel");
  }
  return B200_OK;
}

template <typename QA>
int dispatch_mma(int rank, void* out, int64_t out_hs, int64_t out_ts, float* o_part, float* ml_part, int n_splits,
                 const void* qa, int64_t qa_hs, int64_t qa_ts, const void* q, int64_t ldq, const void* cache,
                 int64_t ldc, const int* q_cu, const int* kv_cu, const int* tables, const int* blk_cu,
                 const int* token_seq, int64_t rows, int H, int dim, int rd, int block_size, float scale,
                 int window, cudaStream_t st) {
#define LM_ARGS out, out_hs, out_ts, o_part, ml_part, n_splits, qa, qa_hs, qa_ts, q, ldq, cache, ldc, q_cu, kv_cu, \
                tables, blk_cu, token_seq, rows, H, dim, rd, rank, block_size, scale, window, st
  const int need = (rank + 31) / 32;   // 8-column tiles per warp (4 warps share the latent columns)
  if (need <= 2) return launch_latent_mma<QA, 2>(LM_ARGS);
  if (need <= 4) return launch_latent_mma<QA, 4>(LM_ARGS);
  if (need <= 8) return launch_latent_mma<QA, 8>(LM_ARGS);
  if (need <= 16) return launch_latent_mma<QA, 16>(LM_ARGS);
#undef LM_ARGS
  return set_error(B200_ERR_UNSUPPORTED, "latent_attn: the tensor-core form takes latent ranks up to 512 (got %d); "
                   "pass n_splits = 0", rank);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t ld_dkv, void* cache, int64_t ldc,
                        const float* c_norm_weight, const float* inv_freq, float mult,
                        const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H,
                        int64_t dim, int64_t rd, int64_t dims, int64_t rank, float eps, int half_pairs, int dtype,
                        b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q && dkv && cache && c_norm_weight && inv_freq && positions && slots,
                 "latent_prepare: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && dim >= 0 && rd >= 0 && rank > 0 && dims >= 0 && dims <= rd &&
                     dims % 2 == 0 && dims <= 4096 && ldq >= H * (dim + rd) && ld_dkv >= rank + rd &&
                     ldc >= rank + rd,
                 "latent_prepare: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)dims * sizeof(float);
#define LP_LAUNCH(T)                                                                                   \
  latent_prepare_kernel<T><<<(unsigned)rows, 128, smem, st>>>(                                          \
      static_cast<T*>(q), ldq, static_cast<const T*>(dkv), ld_dkv, static_cast<T*>(cache), ldc,          \
      c_norm_weight, inv_freq, mult, positions, slots, (int)H, (int)dim, (int)rd, (int)dims, (int)rank, eps,   \
      half_pairs)
  switch (dtype) {
    case B200_BF16: LP_LAUNCH(__nv_bfloat16); break;
    case B200_FP16: LP_LAUNCH(__half); break;
    case B200_FP32: LP_LAUNCH(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef LP_LAUNCH
  B200_LAUNCH_OK("latent_prepare_kernel");
  return B200_OK;
}

int64_t b200_latent_attn_workspace_bytes(int64_t rows, int64_t H, int64_t rank, int64_t n_splits) {
  if (n_splits <= 1) return 0;
  return n_splits * rows * H * (rank + 2) * (int64_t)sizeof(float);
}

int b200_latent_attn(void* out, int64_t out_head_stride, int64_t out_token_stride, const void* q_absorbed,
                     int64_t qa_head_stride, int64_t qa_token_stride, int qa_is_fp32, const void* q,
                     int64_t ldq, const void* cache, int64_t ldc, const int32_t* q_cu_lens,
                     const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                     const int32_t* token_seq, int64_t rows, int64_t H, int64_t dim, int64_t rd,
                     int64_t rank, int64_t block_size, float scale, int64_t window, int n_splits, void* workspace,
                     int64_t workspace_bytes, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q_absorbed && q && cache && q_cu_lens && kv_cu_lens && block_tables &&
                     cu_block_lens && token_seq,
                 "latent_attn: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && H <= 65535 * kHeadsPerCta && dim >= 0 && rd >= 0 && rank > 0 &&
                     block_size > 0 && ldq >= H * (dim + rd) && ldc >= rank + rd && window >= 0 && window < (1ll << 31),
                 "latent_attn: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define LA_CALL(T, QA)                                                                                  \
  return dispatch_nr<T, QA>((int)rank, out, out_head_stride, out_token_stride, q_absorbed, qa_head_stride, \
                            qa_token_stride, q, ldq, cache, ldc, q_cu_lens, kv_cu_lens, block_tables,    \
                            cu_block_lens, token_seq, rows, (int)H, (int)dim, (int)rd, (int)block_size,   \
                            scale, (int)window, st)
  if (dtype == B200_BF16 && n_splits >= 1) {   // tensor-core form
    B200_CHECK_ARG((rank + rd) % 8 == 0 && ldc % 8 == 0 && is_aligned(cache, 16),
                   "latent_attn: the tensor-core form needs 16-byte aligned cache rows (rank + rot_dim and the row "
                   "stride multiples of 8); pass n_splits = 0 for the CUDA-core form");
    B200_CHECK_ARG(n_splits <= 65535, "latent_attn: too many splits");
    float *o_part = nullptr, *ml_part = nullptr;
    if (n_splits > 1) {
      const int64_t need = b200_latent_attn_workspace_bytes(rows, H, rank, n_splits);
      B200_CHECK_ARG(workspace && workspace_bytes >= need && is_aligned(workspace, 16),
                     "latent_attn: workspace of %lld bytes required", (long long)need);
      o_part = static_cast<float*>(workspace);
      ml_part = o_part + (size_t)n_splits * rows * H * rank;
    }
    if (qa_is_fp32)
      return dispatch_mma<float>((int)rank, out, out_head_stride, out_token_stride, o_part, ml_part, n_splits,
                                 q_absorbed, qa_head_stride, qa_token_stride, q, ldq, cache, ldc, q_cu_lens,
                                 kv_cu_lens, block_tables, cu_block_lens, token_seq, rows, (int)H, (int)dim,
                                 (int)rd, (int)block_size, scale, (int)window, st);
    return dispatch_mma<__nv_bfloat16>((int)rank, out, out_head_stride, out_token_stride, o_part, ml_part,
                                       n_splits, q_absorbed, qa_head_stride, qa_token_stride, q, ldq, cache, ldc,
                                       q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, token_seq, rows, (int)H,
                                       (int)dim, (int)rd, (int)block_size, scale, (int)window, st);
  }
  switch (dtype) {
    case B200_BF16:
      if (qa_is_fp32) { LA_CALL(__nv_bfloat16, float); }
      LA_CALL(__nv_bfloat16, __nv_bfloat16);
    case B200_FP32:
      LA_CALL(float, float);
    default:
      return set_error(B200_ERR_UNSUPPORTED, "latent_attn: bf16 or fp32 activations");
  }
#undef LA_CALL
}

}  // extern "C"
