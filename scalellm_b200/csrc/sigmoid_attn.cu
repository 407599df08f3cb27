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
                    float scale, float cap, int size, float* __restrict__ partial) {
  // gridDim.y > 1: CTA (b, s) takes every gridDim.y-th key tile of its rows and leaves its sums in
  // partial[row][s][H * vdim] (the weights are not normalised over the keys, so the shares simply add up)
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

    for (int t0 = j0 + (int)blockIdx.y * KT; t0 <= p_last; t0 += KT * (int)gridDim.y) {
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
          if (r < n) {
            if (partial) partial[((size_t)(run0 + r) * gridDim.y + blockIdx.y) * nout + o] = acc[r][c];
            else out[(size_t)(run0 + r) * ldo + o] = Num<T>::from_f(acc[r][c]);
          }
      }
    }
    run0 += n;
  }
}


// ------------------------------------------------------------------------------------------------------------
// Prompt portions in bf16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
// One CTA = 16 warps = 16 consecutive tokens of one sequence x ALL heads x a range of VW value channels (grid z).
// Keys walk in tiles of 16 from the first key of the first row's block of positions; K [G][16][dim] and the CTA's
// channels of V [G][16][VW] are copied asynchronously through the block table (two buffers where they fit).  Per tile:
//   scores   unit = (head, 8 keys): S = Q K^T, scale, cap, head bias, sigmoid; causal and same-block test per
//            element; the weights go to shared memory in fp32, [head][row][key]
//   mix      unit = (head, part of its channels): the thread gathers its A-fragment positions of
//            a'_h = sum_g M[h, g] a_g from shared memory (fp32) and splits them into two bf16 terms (hi + lo)
//   sum      O_h += a'_h V_g for the unit's channel blocks, both terms
// The queries are rounded to bf16 like the cached keys; everything after the product is fp32.
// ------------------------------------------------------------------------------------------------------------
constexpr int kTW = 16;           // warps per CTA
constexpr int kTK = 16;           // keys per tile
constexpr int kAS = kTK + 1;      // row stride of the weights in shared memory

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

// UPW: (head, part) units a warp owns in the mix and the sum; NPU: blocks of 16 value channels per unit
template <int UPW, int NPU>
__global__ void __launch_bounds__(kTW * 32, 1)
sigmoid_attn_prefill_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                            const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                            const float* __restrict__ head_bias, const float* __restrict__ head_mix,
                            const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                            const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens, int H, int G,
                            int dim, int vdim, int block_size, float scale, float cap, int size, int VW, int parts,
                            int npu, int nbuf) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int KROW = dim + 8, VROW = VW + 8;               // bf16 elements per staged row (16 bytes of padding)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);          // [H][16][KROW]
  __nv_bfloat16* Ks = Qs + (size_t)H * 16 * KROW;                       // [nbuf][G][kTK][KROW] (+ 16 elements slack)
  __nv_bfloat16* Vs = Ks + (size_t)nbuf * G * kTK * KROW + 16;          // [nbuf][G][kTK][VROW]
  float* a_s = reinterpret_cast<float*>(Vs + (size_t)nbuf * G * kTK * VROW);   // [H][16][kAS]
  float* mix_s = a_s + (size_t)H * 16 * kAS;                            // [H][H]
  float* hb_s = mix_s + (head_mix ? H * H : 0);                         // [H]
  const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = q_cu[seq], q_len = q_cu[seq + 1] - q0, kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int t0 = blockIdx.x * 16;                        // first token of the CTA within the step's portion
  if (t0 >= q_len) return;
  const int R = H / G, KS = dim / 16;
  const int ch0 = blockIdx.z * VW;                       // first value channel of this CTA
  const int P0 = kv_len - q_len + t0;                    // position of the CTA's first row
  const int n_rows = min(16, q_len - t0);
  const int P1 = P0 + n_rows - 1;
  const int jb = size > 0 ? (P0 / size) * size : 0;      // first key any row of the CTA sees
  const int n_tiles = (P1 - jb) / kTK + 1;
  const int* table = block_tables + cu_block_lens[seq];
  if (head_mix)
    for (int i = threadIdx.x; i < H * H; i += kTW * 32) mix_s[i] = head_mix[i];
  for (int i = threadIdx.x; i < H; i += kTW * 32) hb_s[i] = head_bias ? head_bias[i] : 0.0f;
  for (int e = threadIdx.x; e < H * 16 * dim; e += kTW * 32) {
    const int d = e % dim, rh = e / dim, rr = rh % 16, h = rh / 16;
    const float v = rr < n_rows ? q[((size_t)(q0 + t0 + rr) * H + h) * dim + d] : 0.0f;
    Qs[((size_t)h * 16 + rr) * KROW + d] = __float2bfloat16_rn(v);
  }
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  const int kchunks = dim / 8, vchunks = VW / 8;
  // a warp takes whole (key/value head, key) rows of the tile: one block-table lookup a row, the lanes copy the row's
  // 16-byte pieces (no division by a runtime number per piece)
  auto load_tile = [&](int idx, int buf) {
    const int per_row = kchunks + vchunks;
    for (int rw = warp; rw < G * kTK; rw += kTW) {
      const int g = rw / kTK, key = rw % kTK;
      const int j = jb + idx * kTK + key;
      const bool ok = j <= P1;
      size_t slot = 0;
      if (ok) slot = (size_t)table[j / block_size] + j % block_size;
      const __nv_bfloat16* ksrc = k_cache + slot * k_stride + (size_t)g * dim;
      const __nv_bfloat16* vsrc = v_cache + slot * v_stride + (size_t)g * vdim + ch0;
      __nv_bfloat16* kdst = Ks + (((size_t)buf * G + g) * kTK + key) * KROW;
      __nv_bfloat16* vdst = Vs + (((size_t)buf * G + g) * kTK + key) * VROW;
      for (int c = lane; c < per_row; c += 32) {
        if (c < kchunks) cp_async16(kdst + c * 8, ksrc + c * 8, ok);
        else cp_async16(vdst + (c - kchunks) * 8, vsrc + (c - kchunks) * 8, ok);
      }
    }
  };
  load_tile(0, 0);
  cp_async_commit();

  const int gr = lane >> 2, qc = (lane & 3) * 2;         // fragment row within 8, first column of the pair
  int pos[2], blk0[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rr = gr + r * 8;
    pos[r] = rr < n_rows ? P0 + rr : -1;
    blk0[r] = (size > 0 && pos[r] >= 0) ? (pos[r] / size) * size : 0;
  }
  const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
  float o[UPW][NPU * 2][4];
#pragma unroll
  for (int u = 0; u < UPW; ++u)
#pragma unroll
    for (int n = 0; n < NPU * 2; ++n) o[u][n][0] = o[u][n][1] = o[u][n][2] = o[u][n][3] = 0.0f;
  const int n_units = H * parts;

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = nbuf == 2 ? (it & 1) : 0;
    cp_async_wait_all();
    __syncthreads();                                     // tile `it` has landed; everyone is done with tile it - 1
    if (nbuf == 2 && it + 1 < n_tiles) {
      load_tile(it + 1, buf ^ 1);
      cp_async_commit();
    }
    const int j0 = jb + it * kTK;
    const __nv_bfloat16* kt = Ks + (size_t)buf * G * kTK * KROW;
    const __nv_bfloat16* vt = Vs + (size_t)buf * G * kTK * VROW;
    // scores: unit = (head, half of the tile's keys)
    for (int u = warp; u < H * 2; u += kTW) {
      const int h = u >> 1, nt = u & 1;
      const __nv_bfloat16* qh = Qs + (size_t)h * 16 * KROW;
      const __nv_bfloat16* kg = kt + (size_t)(h / R) * kTK * KROW;
      float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int ks = 0; ks < KS; ks += 2) {
        uint32_t a[4], b[4];
        ldsm_x4(b, kg + (nt * 8 + (lane & 7)) * KROW + ks * 16 + (lane >> 3) * 8);
        ldsm_x4(a, qh + (lane & 15) * KROW + ks * 16 + (lane >> 4) * 8);
        mma_bf16(sc, a, b[0], b[1]);
        if (ks + 1 < KS) {
          ldsm_x4(a, qh + (lane & 15) * KROW + (ks + 1) * 16 + (lane >> 4) * 8);
          mma_bf16(sc, a, b[2], b[3]);
        }
      }
      const float hb = hb_s[h];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int j = j0 + nt * 8 + qc + (e & 1);
        float w = 0.0f;
        if (j <= pos[r] && j >= blk0[r]) {
          // cap and sigmoid through the fast exponential (absolute error of tanh about 1e-7: far below the rounding
          // of the 16-bit keys); the plain functions were a third of this kernel's instructions
          float v = sc[e] * scale;
          if (cap > 0.0f) v = cap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v * inv_cap)));
          w = __fdividef(1.0f, 1.0f + __expf(-(v + hb)));
        }
        a_s[((size_t)h * 16 + gr + r * 8) * kAS + nt * 8 + qc + (e & 1)] = w;
      }
    }
    __syncthreads();
    // mix and weighted sum: unit = (head, part of the CTA's channels)
#pragma unroll
    for (int uu = 0; uu < UPW; ++uu) {
      const int u = warp + uu * kTW;
      if (u < n_units) {
        const int h = u / parts, part = u - h * parts;
        float m[8];                                       // (row gr | gr + 8) x (keys qc, qc + 1 | qc + 8, qc + 9)
#pragma unroll
        for (int i = 0; i < 8; ++i) m[i] = 0.0f;
        if (head_mix) {
          for (int g2 = 0; g2 < H; ++g2) {
            const float t = mix_s[h * H + g2];
            const float* ar = a_s + (size_t)g2 * 16 * kAS;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              m[i] += t * ar[(gr + ((i >> 1) & 1) * 8) * kAS + qc + (i & 1) + (i >> 2) * 8];
          }
        } else {
          const float* ar = a_s + (size_t)h * 16 * kAS;
#pragma unroll
          for (int i = 0; i < 8; ++i) m[i] = ar[(gr + ((i >> 1) & 1) * 8) * kAS + qc + (i & 1) + (i >> 2) * 8];
        }
        uint32_t phi[4], plo[4];
        split_bf16(m[0], m[1], phi[0], plo[0]);           // a0: row gr, keys qc..
        split_bf16(m[2], m[3], phi[1], plo[1]);           // a1: row gr + 8
        split_bf16(m[4], m[5], phi[2], plo[2]);           // a2: row gr, keys qc + 8..
        split_bf16(m[6], m[7], phi[3], plo[3]);           // a3: row gr + 8
        const __nv_bfloat16* vg = vt + (size_t)(h / R) * kTK * VROW;
        const __nv_bfloat16* vrow = vg + ((lane & 7) + ((lane >> 3) & 1) * 8) * VROW + (lane >> 4) * 8;
#pragma unroll
        for (int n = 0; n < NPU; ++n) {
          const int cb = part * npu + n;                  // block of 16 channels within the CTA's range
          if (n < npu && cb * 16 < VW) {
            uint32_t b[4];
            ldsm_x4_t(b, vrow + cb * 16);
            mma_bf16(o[uu][n * 2], phi, b[0], b[1]);
            mma_bf16(o[uu][n * 2 + 1], phi, b[2], b[3]);
            mma_bf16(o[uu][n * 2], plo, b[0], b[1]);
            mma_bf16(o[uu][n * 2 + 1], plo, b[2], b[3]);
          }
        }
      }
    }
    if (nbuf == 1 && it + 1 < n_tiles) {
      __syncthreads();                                   // the single buffer is free again
      load_tile(it + 1, 0);
      cp_async_commit();
    }
  }
  cp_async_wait_all();
#pragma unroll
  for (int uu = 0; uu < UPW; ++uu) {
    const int u = warp + uu * kTW;
    if (u >= n_units) continue;
    const int h = u / parts, part = u - h * parts;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (pos[r] < 0) continue;
      __nv_bfloat16* dst = out + (size_t)(q0 + t0 + gr + r * 8) * ldo + (size_t)h * vdim + ch0;
#pragma unroll
      for (int n = 0; n < NPU * 2; ++n) {
        const int c = (part * npu + (n >> 1)) * 16 + (n & 1) * 8 + qc;
        if ((n >> 1) < npu && c < VW)
          *reinterpret_cast<uint32_t*>(dst + c) = Num<__nv_bfloat16>::pack(o[uu][n][r * 2], o[uu][n][r * 2 + 1]);
      }
    }
  }
}

struct PrefillPlan {
  int zs, VW, parts, npu, upw, nbuf;
  size_t smem;
  bool ok;
};

// The channel split over CTAs, the (head, part) units and the buffers that fit: at most 8 blocks of 16 channels per
// warp (64 accumulator registers), shared memory within the opt-in limit.
inline PrefillPlan plan_prefill(int H, int G, int dim, int vdim, bool mix) {
  PrefillPlan p{};
  p.ok = false;
  if (dim % 16 || vdim % 16 || H % G || dim > 256) return p;
  for (int zs = 1; zs <= 8; zs *= 2) {
    if (vdim % (16 * zs)) break;
    const int VW = vdim / zs, nth = VW / 16;
    int parts = 1;
    while (parts * 2 * H <= kTW && parts * 2 <= nth) parts *= 2;
    const int npu = (nth + parts - 1) / parts;
    const int upw = (H * parts + kTW - 1) / kTW;
    if (upw * npu > 8 || upw > 4) continue;
    for (int nbuf = 2; nbuf >= 1; --nbuf) {
      const size_t smem = ((size_t)H * 16 * (dim + 8) + (size_t)nbuf * G * kTK * (dim + 8) + 16 +
                           (size_t)nbuf * G * kTK * (VW + 8)) * 2 +
                          ((size_t)H * 16 * kAS + (mix ? (size_t)H * H : 0) + H) * 4;
      if (smem <= 227 * 1024) {
        p = PrefillPlan{zs, VW, parts, npu, upw, nbuf, smem, true};
        return p;
      }
    }
  }
  return p;
}

template <int UPW, int NPU>
int launch_prefill(const PrefillPlan& p, void* out, int64_t ldo, const float* q, const void* kc, const void* vc,
                   const float* hb, const float* mix, const int* q_cu, const int* kv_cu, const int* bt, const int* cbl,
                   int64_t n_seq, int64_t q_max, int H, int G, int dim, int vdim, int bs, float scale, float cap,
                   int size, cudaStream_t st) {
  auto kern = sigmoid_attn_prefill_kernel<UPW, NPU>;
  if (p.smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
  dim3 grid((unsigned)((q_max + 15) / 16), (unsigned)n_seq, (unsigned)p.zs);
  kern<<<grid, kTW * 32, p.smem, st>>>(static_cast<__nv_bfloat16*>(out), ldo, q,
                                       static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc),
                                       hb, mix, q_cu, kv_cu, bt, cbl, H, G, dim, vdim, bs, scale, cap, size, p.VW,
                                       p.parts, p.npu, p.nbuf);
  B200_LAUNCH_OK("sigmoid_attn_prefill_kernel");
  return B200_OK;
}

template <typename T>
__global__ void sigmoid_attn_sum_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ partial, int nout,
                                        int n_splits) {
  const int row = blockIdx.x;
  for (int o = threadIdx.x; o < nout; o += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < n_splits; ++s) acc += partial[((size_t)row * n_splits + s) * nout + o];
    out[(size_t)row * ldo + o] = Num<T>::from_f(acc);
  }
}


// Single rows (decoding) with vector loads: one CTA per (row, share of the row's key tiles).
//   scores : 16 lanes per (key, key/value head): one 16-byte load a lane, the dot products with the group's R query
//            heads, a butterfly over the 16 lanes
//   mix    : thread = (head, key), as above
//   sum    : thread = (key/value head, 16 bytes of value channels, one of KG key groups): R x EPV sums in registers;
//            the KG groups are added up through shared memory at the end
// dim and vdim multiples of EPV = 16 / sizeof(T), at most 256 (head, chunk) items, R <= RMAX.
template <typename T, int RMAX>
__global__ void __launch_bounds__(kAttnThreads)
sigmoid_attn_decode_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                           const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                           const float* __restrict__ head_bias, const float* __restrict__ head_mix,
                           const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                           const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens,
                           const int* __restrict__ token_seq, int H, int G, int dim, int vdim, int block_size,
                           float scale, float cap, int size, float* __restrict__ partial) {
  constexpr int EPV = 16 / (int)sizeof(T);
  extern __shared__ __align__(16) float sm[];
  const int R = H / G;
  const int NI = G * (vdim / EPV);                       // (key/value head, chunk) items of the sum
  const int KG = kAttnThreads / NI;                      // key groups
  const int QROW = dim + (dim / 32) * 4;                 // four floats of padding per 32: the 16 lanes' 16-byte reads
                                                         // of one head fall on distinct banks
  float* q_s = sm;                                       // [H][QROW]
  float* a_s = q_s + (size_t)H * QROW;                   // [H][KT]
  float* m_s = a_s + (size_t)H * KT;                     // [H][KT]
  float* mix_s = m_s + (size_t)H * KT;                   // [H][H]
  float* hb_s = mix_s + (head_mix ? H * H : 0);          // [H]
  float* red_s = hb_s + H;                               // [KG][NI][R][EPV]
  __shared__ int slot_s[KT];
  const int row = blockIdx.x;
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int p = kv_len - q_len + (row - q_cu[seq]);      // position of the row
  const int j0 = size > 0 ? (p / size) * size : 0;
  const int* table = block_tables + cu_block_lens[seq];
  const size_t k_stride = (size_t)G * dim, v_stride = (size_t)G * vdim;
  if (head_mix)
    for (int i = threadIdx.x; i < H * H; i += kAttnThreads) mix_s[i] = head_mix[i];
  for (int i = threadIdx.x; i < H; i += kAttnThreads) hb_s[i] = head_bias ? head_bias[i] : 0.0f;
  for (int i = threadIdx.x; i < H * dim; i += kAttnThreads) {
    const int h = i / dim, d = i - h * dim;
    q_s[h * QROW + d + (d / 32) * 4] = q[(size_t)row * H * dim + i];
  }
  const int item = threadIdx.x % NI, kq = threadIdx.x / NI;     // kq >= KG: the thread has no part in the sum
  const int ig = item / (vdim / EPV), ich = item % (vdim / EPV);
  float acc[RMAX][EPV];
#pragma unroll
  for (int r = 0; r < RMAX; ++r)
#pragma unroll
    for (int e = 0; e < EPV; ++e) acc[r][e] = 0.0f;
  const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15;        // 16-lane group and lane within it
  for (int t0 = j0 + (int)blockIdx.y * KT; t0 <= p; t0 += KT * (int)gridDim.y) {
    const int nk = min(KT, p + 1 - t0);
    __syncthreads();                                             // tile before consumed; q_s visible
    if (threadIdx.x < KT) {
      const int j = t0 + min((int)threadIdx.x, nk - 1);
      slot_s[threadIdx.x] = table[j / block_size] + j % block_size;
    }
    __syncthreads();
    // both 16-lane groups of a warp make the same number of rounds (the butterflies take the whole warp); a round
    // takes UB units a group, all their loads issued before the first product, so that a CTA has several loads in
    // flight per thread (the walk is bound by the latency of its loads, not by their number)
    constexpr int UB = 4;
    for (int ub = hw & ~1; ub < nk * G; ub += UB * (kAttnThreads / 16)) {
      bool ok[UB];
      int jj[UB], g[UB];
      float part[UB][RMAX];
#pragma unroll
      for (int i = 0; i < UB; ++i) {
        const int u = ub + i * (kAttnThreads / 16) + (hw & 1);
        ok[i] = u < nk * G;
        const int uu = ok[i] ? u : 0;
        jj[i] = uu / G;
        g[i] = uu - jj[i] * G;
#pragma unroll
        for (int r = 0; r < RMAX; ++r) part[i][r] = 0.0f;
      }
      for (int d = hl * EPV; d < dim; d += 16 * EPV) {
        uint4 raw[UB];
#pragma unroll
        for (int i = 0; i < UB; ++i)
          raw[i] = ok[i] ? ld_nc_v4(k_cache + (size_t)slot_s[jj[i]] * k_stride + (size_t)g[i] * dim + d)
                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < UB; ++i) {
          float kv[EPV];
          if constexpr (sizeof(T) == 4) {
            kv[0] = __uint_as_float(raw[i].x); kv[1] = __uint_as_float(raw[i].y);
            kv[2] = __uint_as_float(raw[i].z); kv[3] = __uint_as_float(raw[i].w);
          } else {
            const uint32_t w4[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 f = Num<T>::unpack(w4[c]);
              kv[2 * c] = f.x;
              kv[2 * c + 1] = f.y;
            }
          }
#pragma unroll
          for (int r = 0; r < RMAX; ++r)
            if (r < R) {
              const float* qh = q_s + (size_t)(g[i] * R + r) * QROW + d + (d / 32) * 4;
#pragma unroll
              for (int e = 0; e < EPV; e += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(qh + e);
                part[i][r] += q4.x * kv[e] + q4.y * kv[e + 1] + q4.z * kv[e + 2] + q4.w * kv[e + 3];
              }
            }
        }
      }
#pragma unroll
      for (int i = 0; i < UB; ++i)
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) part[i][r] += __shfl_xor_sync(0xffffffffu, part[i][r], o);
          if (ok[i] && r < R && hl == 0) a_s[(g[i] * R + r) * KT + jj[i]] = part[i][r];     // the raw product
        }
    }
    __syncthreads();
    // cap, bias and sigmoid with every lane at work (one lane per product would leave 15 of 16 idle)
    for (int i = threadIdx.x; i < H * KT; i += kAttnThreads) {
      const int h = i / KT;
      float w = 0.0f;
      if (i - h * KT < nk) {
        float sc = a_s[i] * scale;
        if (cap > 0.0f) sc = cap * tanhf(sc / cap);
        w = sigmoidf_(sc + hb_s[h]);
      }
      a_s[i] = w;
    }
    __syncthreads();
    const float* w_s = a_s;
    if (head_mix) {
      for (int i = threadIdx.x; i < H * KT; i += kAttnThreads) {
        const int jj = i % KT, h = i / KT;
        float m = 0.0f;
        for (int g2 = 0; g2 < H; ++g2) m += mix_s[h * H + g2] * a_s[g2 * KT + jj];
        m_s[i] = m;
      }
      __syncthreads();
      w_s = m_s;
    }
    if (kq < KG) {
      const T* vb = v_cache + (size_t)ig * vdim + (size_t)ich * EPV;
      for (int jb = kq; jb < nk; jb += UB * KG) {          // UB keys a round, loads first
        uint4 raw[UB];
#pragma unroll
        for (int i = 0; i < UB; ++i) {
          const int jj = jb + i * KG;
          raw[i] = jj < nk ? ld_nc_v4(vb + (size_t)slot_s[jj] * v_stride) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < UB; ++i) {
          const int jj = jb + i * KG;
          if (jj < nk) {
            float vv[EPV];
            if constexpr (sizeof(T) == 4) {
              vv[0] = __uint_as_float(raw[i].x); vv[1] = __uint_as_float(raw[i].y);
              vv[2] = __uint_as_float(raw[i].z); vv[3] = __uint_as_float(raw[i].w);
            } else {
              const uint32_t w4[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const float2 f = Num<T>::unpack(w4[c]);
                vv[2 * c] = f.x;
                vv[2 * c + 1] = f.y;
              }
            }
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
              if (r < R) {
                const float w = w_s[(ig * R + r) * KT + jj];
#pragma unroll
                for (int e = 0; e < EPV; ++e) acc[r][e] += w * vv[e];
              }
          }
        }
      }
    }
  }
  __syncthreads();
  if (kq < KG) {
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
      if (r < R) {
#pragma unroll
        for (int e = 0; e < EPV; ++e) red_s[(((size_t)kq * NI + item) * R + r) * EPV + e] = acc[r][e];
      }
  }
  __syncthreads();
  const int nout = H * vdim;
  for (int o = threadIdx.x; o < nout; o += kAttnThreads) {
    const int h = o / vdim, c = o - h * vdim;
    const int g = h / R, r = h - g * R, it = g * (vdim / EPV) + c / EPV, e = c % EPV;
    float sum = 0.0f;
    for (int k2 = 0; k2 < KG; ++k2) sum += red_s[(((size_t)k2 * NI + it) * R + r) * EPV + e];
    if (partial) partial[((size_t)row * gridDim.y + blockIdx.y) * nout + o] = sum;
    else out[(size_t)row * ldo + o] = Num<T>::from_f(sum);
  }
}

template <typename T>
bool decode_vec_ok(int H, int G, int dim, int vdim, const void* kc, const void* vc) {
  constexpr int EPV = 16 / (int)sizeof(T);
  const int R = H / G;
  return dim % EPV == 0 && vdim % EPV == 0 && G * (vdim / EPV) <= kAttnThreads && R <= 8 && is_aligned(kc, 16) &&
         is_aligned(vc, 16);
}

template <typename T>
int launch_decode_vec(void* out, int64_t ldo, const float* q, const void* kc, const void* vc, const float* hb,
                      const float* mix, const int* q_cu, const int* kv_cu, const int* bt, const int* cbl, const int* ts,
                      int64_t rows, int H, int G, int dim, int vdim, int bs, float scale, float cap, int size,
                      int n_splits, float* partial, cudaStream_t st) {
  constexpr int EPV = 16 / (int)sizeof(T);
  const int R = H / G, NI = G * (vdim / EPV), KG = kAttnThreads / NI;
  const size_t smem = ((size_t)H * (dim + (dim / 32) * 4) + 2 * (size_t)H * KT + (mix ? (size_t)H * H : 0) + H +
                       (size_t)KG * NI * R * EPV) * sizeof(float);
  if (smem > 200 * 1024) return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: %zu bytes of shared memory", smem);
  const dim3 grid((unsigned)rows, (unsigned)n_splits);
#define SD_LAUNCH(RM)                                                                                               \
  do {                                                                                                              \
    auto kern = sigmoid_attn_decode_kernel<T, RM>;                                                                  \
    if (smem > 48 * 1024)                                                                                           \
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));             \
    kern<<<grid, kAttnThreads, smem, st>>>(static_cast<T*>(out), ldo, q, static_cast<const T*>(kc),                 \
                                           static_cast<const T*>(vc), hb, mix, q_cu, kv_cu, bt, cbl, ts, H, G, dim, \
                                           vdim, bs, scale, cap, size, n_splits > 1 ? partial : nullptr);           \
  } while (0)
  if (R <= 1) SD_LAUNCH(1);
  else if (R <= 2) SD_LAUNCH(2);
  else if (R <= 4) SD_LAUNCH(4);
  else SD_LAUNCH(8);
#undef SD_LAUNCH
  B200_LAUNCH_OK("sigmoid_attn_decode_kernel");
  if (n_splits > 1) {
    sigmoid_attn_sum_kernel<T><<<(unsigned)rows, 256, 0, st>>>(static_cast<T*>(out), ldo, partial, H * vdim, n_splits);
    B200_LAUNCH_OK("sigmoid_attn_sum_kernel");
  }
  return B200_OK;
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
                int n_splits, float* partial, cudaStream_t st) {
  if constexpr (NC * RQ > 32) {
    return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: %d sums per thread", NC * RQ);
  } else {
  const size_t smem = ((size_t)RQ * H * dim + 2 * (size_t)RQ * H * KT + (mix ? (size_t)H * H : 0) + H) * sizeof(float);
  if (smem > 200 * 1024) return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn: %zu bytes of shared memory", smem);
  auto kern = sigmoid_attn_kernel<T, NC, RQ>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const dim3 grid((unsigned)((rows + RQ - 1) / RQ), (unsigned)n_splits);
  kern<<<grid, kAttnThreads, smem, st>>>(static_cast<T*>(out), ldo, q, static_cast<const T*>(kc),
                                         static_cast<const T*>(vc), hb, mix, q_cu, kv_cu, bt, cbl, ts, (int)rows, H,
                                         G, dim, vdim, bs, scale, cap, size, n_splits > 1 ? partial : nullptr);
  B200_LAUNCH_OK("sigmoid_attn_kernel");
  if (n_splits > 1) {
    sigmoid_attn_sum_kernel<T><<<(unsigned)rows, 256, 0, st>>>(static_cast<T*>(out), ldo, partial, H * vdim, n_splits);
    B200_LAUNCH_OK("sigmoid_attn_sum_kernel");
  }
  return B200_OK;
  }
}

template <typename T, int RQ>
int launch_attn_nc(int nc, void* out, int64_t ldo, const float* q, const void* kc, const void* vc, const float* hb,
                   const float* mix, const int* q_cu, const int* kv_cu, const int* bt, const int* cbl, const int* ts,
                   int64_t rows, int H, int G, int dim, int vdim, int bs, float scale, float cap, int size,
                   int n_splits, float* partial, cudaStream_t st) {
#define SA_NC(N)                                                                                                  \
  return launch_attn<T, N, RQ>(out, ldo, q, kc, vc, hb, mix, q_cu, kv_cu, bt, cbl, ts, rows, H, G, dim, vdim, bs, \
                               scale, cap, size, n_splits, partial, st)
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
                      int64_t block_size, float scale, float cap, int64_t size, int64_t rows_per_cta,
                      int64_t n_splits, float* workspace, int64_t workspace_floats, int dtype, b200_stream_t stream) {
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
  if (n_splits < 1 || rq > 1) n_splits = 1;       // key tiles are shared out over CTAs for single rows only
  B200_CHECK_ARG(n_splits == 1 || (workspace && workspace_floats >= rows * n_splits * H * vdim && n_splits <= 65535),
                 "sigmoid_attn: the workspace takes rows * n_splits * H * vdim floats");
  if (rq == 1) {
    SA_DISPATCH(dtype, {
      if (decode_vec_ok<T>((int)H, (int)G, (int)dim, (int)vdim, k_cache, v_cache))
        return launch_decode_vec<T>(out, ldo, q, k_cache, v_cache, head_bias, head_mix, q_cu_lens, kv_cu_lens,
                                    block_tables, cu_block_lens, token_seq, rows, (int)H, (int)G, (int)dim, (int)vdim,
                                    (int)block_size, scale, cap, (int)size, (int)n_splits, workspace, st);
    });
  }
#define SA_RQ(N)                                                                                                     \
  SA_DISPATCH(dtype, return (launch_attn_nc<T, N>(nc, out, ldo, q, k_cache, v_cache, head_bias, head_mix, q_cu_lens, \
                                                  kv_cu_lens, block_tables, cu_block_lens, token_seq, rows, (int)H,  \
                                                  (int)G, (int)dim, (int)vdim, (int)block_size, scale, cap,          \
                                                  (int)size, (int)n_splits, workspace, st)))
  if (rq >= 8) { SA_RQ(8); }
  if (rq >= 4) { SA_RQ(4); }
  if (rq >= 2) { SA_RQ(2); }
  SA_RQ(1);
#undef SA_RQ
  return B200_OK;
}

int b200_sigmoid_attn_prefill_supported(int64_t H, int64_t G, int64_t dim, int64_t vdim, int has_mix, int dtype) {
  if (dtype != B200_BF16 || H <= 0 || G <= 0) return 0;
  return plan_prefill((int)H, (int)G, (int)dim, (int)vdim, has_mix != 0).ok ? 1 : 0;
}

int b200_sigmoid_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                              const float* head_bias, const float* head_mix, const int32_t* q_cu_lens,
                              const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                              int64_t n_seq, int64_t q_max, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                              int64_t block_size, float scale, float cap, int64_t size, int dtype,
                              b200_stream_t stream) {
  if (n_seq == 0 || q_max == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens,
                 "sigmoid_attn_prefill: null pointer");
  B200_CHECK_ARG(dtype == B200_BF16 && n_seq > 0 && q_max > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 &&
                     ldo >= H * vdim && size >= 0 && size < (1ll << 31) && ldo % 2 == 0,
                 "sigmoid_attn_prefill: bad shape (bf16 only)");
  const PrefillPlan p = plan_prefill((int)H, (int)G, (int)dim, (int)vdim, head_mix != nullptr);
  if (!p.ok) return set_error(B200_ERR_UNSUPPORTED, "sigmoid_attn_prefill: sizes %d x %d / %d heads do not fit",
                              (int)dim, (int)vdim, (int)H);
  auto st = static_cast<cudaStream_t>(stream);
#define SP_ARGS p, out, ldo, q, k_cache, v_cache, head_bias, head_mix, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, \
                n_seq, q_max, (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, cap, (int)size, st
  if (p.upw == 1 && p.npu <= 4) return launch_prefill<1, 4>(SP_ARGS);
  if (p.upw == 1) return launch_prefill<1, 8>(SP_ARGS);
  if (p.upw == 2 && p.npu <= 4) return launch_prefill<2, 4>(SP_ARGS);
  return launch_prefill<4, 2>(SP_ARGS);
#undef SP_ARGS
}

}  // extern "C"
