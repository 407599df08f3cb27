// moe.cu — token-choice mixture of experts: router, expert plan, grouped GEMM, combine.
//
//   route    z = Wr h in fp32 (Wr kept in fp32), s = sigmoid(z); the `top` largest per token are
//            chosen (first index wins a tie); the routing weight of a choice is s itself.
//   plan     counting sort of the (token, choice) pairs by expert: offsets[E + 1], the pair at each
//            sorted position and the sorted position of each pair — all on the device, so a step
//            never synchronises with the host.
//   grouped  C[pos, :] = A(pos) W_e^T for every sorted position of expert e.  A(pos) is either row
//            pos of a sorted activation matrix, or (gather form) the routing weight times the
//            token's input row: the weight scales what the expert reads, not what it returns.
//            64 x 64 tiles, fp32 accumulation in k order: a row's result does not depend on where
//            the row sits in a tile or on what shares the tile.
//   combine  out[t] = sum over choices of Y[position of (t, choice)], summed in choice order.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTop = 32;
constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(int* __restrict__ ids, float* __restrict__ weights, const T* __restrict__ h, int64_t ldh,
                 const float* __restrict__ Wr, int W, int E, int top) {
  __shared__ float z_s[kMaxExperts];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* x = h + (size_t)row * ldh;
  for (int e = warp; e < E; e += 4) {
    const float* w = Wr + (size_t)e * W;
    float acc = 0.0f;
    for (int i = lane; i < W; i += 32) acc += Num<T>::to_f(x[i]) * w[i];
    acc = warp_sum(acc);
    if (lane == 0) z_s[e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 0; k < top; ++k) {
      int best = 0;
      float bz = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float z = z_s[e];
        if (z > bz) { bz = z; best = e; }
      }
      ids[(size_t)row * top + k] = best;
      weights[(size_t)row * top + k] = 1.0f / (1.0f + expf(-bz));
      z_s[best] = -INFINITY;
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ offsets, int* __restrict__ sorted_pair, int* __restrict__ pos_of_pair,
                const int* __restrict__ ids, int n_pairs, int E) {
  __shared__ int cnt[kMaxExperts + 1];
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      offsets[e] = run;
      cnt[e] = run;
      run += c;
    }
    offsets[E] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int pos = atomicAdd(&cnt[ids[p]], 1);
    sorted_pair[pos] = p;
    pos_of_pair[p] = pos;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(T* __restrict__ C, int64_t ldc, const T* __restrict__ A, int64_t lda,
                    const int* __restrict__ sorted_pair, const float* __restrict__ pair_scale, int top,
                    const T* __restrict__ Wst, const int* __restrict__ offsets, int E, int N, int K) {
  __shared__ float As[BK][BM + 4], Bs[BK][BN + 4];
  __shared__ int src_row[BM];
  __shared__ float src_scale[BM];
  // which expert and which of its row tiles is this CTA's
  int e = 0, tile = blockIdx.y, lo = 0, hi = 0;
  for (; e < E; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int nt = (hi - lo + BM - 1) / BM;
    if (tile < nt) break;
    tile -= nt;
  }
  if (e == E) return;
  const int m0 = lo + tile * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < BM) {
    const int pos = m0 + tid;
    int src = -1;
    float sc = 1.0f;
    if (pos < hi) {
      if (sorted_pair) {
        const int p = sorted_pair[pos];
        src = p / top;
        sc = pair_scale ? pair_scale[p] : 1.0f;
      } else {
        src = pos;
      }
    }
    src_row[tid] = src;
    src_scale[tid] = sc;
  }
  __syncthreads();
  const T* Wm = Wst + (size_t)e * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + 256 * i;
      const int m = idx >> 4, kk = idx & 15;
      const int src = src_row[m];
      float a = 0.0f, b = 0.0f;
      if (k0 + kk < K) {
        if (src >= 0) a = Num<T>::to_f(A[(size_t)src * lda + k0 + kk]) * src_scale[m];
        if (n0 + m < N) b = Num<T>::to_f(Wm[(size_t)(n0 + m) * K + k0 + kk]);
      }
      As[kk][m] = a;
      Bs[kk][m] = b;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int pos = m0 + ty * 4 + i;
    if (pos >= hi) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)pos * ldc + n] = Num<T>::from_f(acc[i][j]);
    }
  }
}


// Few rows per expert (decoding): the weights are the traffic.  One CTA per (expert, 16 output columns):
// the expert's rows, MB at a time, sit in shared memory; every warp streams two weight rows at a time with
// 16-byte loads and keeps MB x 2 dot products per lane, reduced over the warp at the end.  Sums run in k
// order per lane and then over lanes: a row's result does not depend on which rows share its pass.
constexpr int GV_MB = 8, GV_WARPS = 8, GV_CPW = 2;

template <typename T>
__global__ void __launch_bounds__(GV_WARPS * 32)
grouped_gemv_kernel(T* __restrict__ C, int64_t ldc, const T* __restrict__ A, int64_t lda,
                    const int* __restrict__ sorted_pair, const float* __restrict__ pair_scale, int top,
                    const T* __restrict__ Wst, const int* __restrict__ offsets, int N, int K) {
  extern __shared__ __align__(16) unsigned char gv_smem[];
  T* As = reinterpret_cast<T*>(gv_smem);                     // [GV_MB][K]
  constexpr int VEC = 16 / sizeof(T);
  const int e = blockIdx.y, lo = offsets[e], hi = offsets[e + 1];
  if (lo >= hi) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_CPW;
  const T* Wm = Wst + (size_t)e * N * K;
  for (int m0 = lo; m0 < hi; m0 += GV_MB) {
    __syncthreads();
    for (int m = 0; m < GV_MB; ++m) {
      const int pos = m0 + m;
      int src = -1;
      float sc = 1.0f;
      if (pos < hi) {
        if (sorted_pair) {
          const int p = sorted_pair[pos];
          src = p / top;
          sc = pair_scale ? pair_scale[p] : 1.0f;
        } else {
          src = pos;
        }
      }
      for (int k = threadIdx.x; k < K; k += GV_WARPS * 32)
        As[m * K + k] = src >= 0 ? Num<T>::from_f(Num<T>::to_f(A[(size_t)src * lda + k]) * sc) : Num<T>::from_f(0.0f);
    }
    __syncthreads();
    if (n0 < N) {
      float acc[GV_CPW][GV_MB];
#pragma unroll
      for (int c = 0; c < GV_CPW; ++c)
#pragma unroll
        for (int m = 0; m < GV_MB; ++m) acc[c][m] = 0.0f;
      for (int k = lane * VEC; k < K; k += 32 * VEC) {
        T w[GV_CPW][VEC];
#pragma unroll
        for (int c = 0; c < GV_CPW; ++c) {
          const int n = n0 + c < N ? n0 + c : N - 1;
          *reinterpret_cast<uint4*>(w[c]) = *reinterpret_cast<const uint4*>(Wm + (size_t)n * K + k);
        }
#pragma unroll
        for (int m = 0; m < GV_MB; ++m) {
          T a[VEC];
          *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(As + m * K + k);
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            const float av = Num<T>::to_f(a[v]);
#pragma unroll
            for (int c = 0; c < GV_CPW; ++c) acc[c][m] += av * Num<T>::to_f(w[c][v]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < GV_CPW; ++c)
#pragma unroll
        for (int m = 0; m < GV_MB; ++m) {
          const float v = warp_sum(acc[c][m]);
          if (lane == 0 && n0 + c < N && m0 + m < hi) C[(size_t)(m0 + m) * ldc + n0 + c] = Num<T>::from_f(v);
        }
    }
  }
}

// xs[pos] = pair_scale[pair] * h[pair / top]: the experts' input rows in sorted order (for a library grouped GEMM)
template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ h, int64_t ldh,
                                  const int* __restrict__ sorted_pair, const float* __restrict__ pair_scale,
                                  int top, int W) {
  const int pos = blockIdx.x, p = sorted_pair[pos];
  const float sc = pair_scale ? pair_scale[p] : 1.0f;
  const T* src = h + (size_t)(p / top) * ldh;
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[(size_t)pos * W + i] = Num<T>::from_f(Num<T>::to_f(src[i]) * sc);
}

// out[row] = scale * sum_k Y[pos_of_pair[row, k]] (+ addend[row]: a result every token gets, a shared expert's)
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ Y, int64_t ldy,
                                   const int* __restrict__ pos_of_pair, int W, int top, float scale,
                                   const T* __restrict__ addend, int64_t ld_add) {
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k)
      acc += Num<T>::to_f(Y[(size_t)pos_of_pair[(size_t)row * top + k] * ldy + i]);
    acc *= scale;
    if (addend) acc += Num<T>::to_f(addend[(size_t)row * ld_add + i]);
    out[(size_t)row * W + i] = Num<T>::from_f(acc);
  }
}

// ids[row, k] = table[token of the row, k]: the experts of a token are a property of its id
__global__ void moe_table_route_kernel(int* __restrict__ ids, const int* __restrict__ table,
                                       const int* __restrict__ tokens, int64_t n, int top, int vocab, int E) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int tok = tokens[i / top];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    int e = table[(int64_t)tok * top + i % top];
    ids[i] = e < 0 ? 0 : (e >= E ? E - 1 : e);
  }
}

// Softmax router with a choice correction and a limit to the best groups:
//     p = softmax(Wr h) over the E outputs (fp32) ;  c = p + correction
//     the E outputs form n_groups equal runs of neighbours; a run's score is its largest c; outside the keep_groups
//     best runs c counts as -inf
//     the `top` largest c are chosen (first index wins a tie); weight = p / (sum of the chosen p + weight_eps)
// extra_w (nullable): one more row for the same input, extra_out[row] = sigmoid(extra_w . h) (a gate every token gets).
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_softmax_kernel(int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ extra_out,
                         const T* __restrict__ h, int64_t ldh, const float* __restrict__ Wr,
                         const float* __restrict__ correction, const float* __restrict__ extra_w, int W, int E,
                         int top, int n_groups, int keep_groups, float weight_eps) {
  __shared__ float z_s[kMaxExperts + 1];     // logits, then probabilities
  __shared__ float c_s[kMaxExperts];         // choice scores
  __shared__ unsigned char dead[kMaxExperts];
  __shared__ float red[32];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* x = h + (size_t)row * ldh;
  const int n_dots = E + (extra_w ? 1 : 0);
  for (int e = warp; e < n_dots; e += 4) {
    const float* w = e < E ? Wr + (size_t)e * W : extra_w;
    float acc = 0.0f;
    for (int i = lane; i < W; i += 32) acc += Num<T>::to_f(x[i]) * w[i];
    acc = warp_sum(acc);
    if (lane == 0) z_s[e] = acc;
  }
  __syncthreads();
  if (extra_w && threadIdx.x == 0) extra_out[row] = 1.0f / (1.0f + expf(-z_s[E]));
  float mx = -INFINITY;
  for (int e = threadIdx.x; e < E; e += 128) mx = fmaxf(mx, z_s[e]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.0f;
  for (int e = threadIdx.x; e < E; e += 128) {
    const float ex = expf(z_s[e] - mx);
    z_s[e] = ex;
    sum += ex;
  }
  sum = block_sum<128>(sum, red);
  for (int e = threadIdx.x; e < E; e += 128) {
    const float p = z_s[e] / sum;
    z_s[e] = p;
    c_s[e] = p + (correction ? correction[e] : 0.0f);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (n_groups > 1 && keep_groups < n_groups) {
      const int gs = E / n_groups;
      // drop the worst n_groups - keep_groups runs: repeatedly find the live run with the smallest score (the last
      // index loses a tie, as the first index wins among the kept)
      for (int g = 0; g < n_groups; ++g) dead[g] = 0;
      for (int k = 0; k < n_groups - keep_groups; ++k) {
        int worst = -1;
        float wz = INFINITY;
        for (int g = 0; g < n_groups; ++g) {
          if (dead[g]) continue;
          float best = -INFINITY;
          for (int e = g * gs; e < (g + 1) * gs; ++e) best = fmaxf(best, c_s[e]);
          if (best <= wz) { wz = best; worst = g; }
        }
        dead[worst] = 1;
      }
      for (int g = 0; g < n_groups; ++g)
        if (dead[g])
          for (int e = g * gs; e < (g + 1) * gs; ++e) c_s[e] = -INFINITY;
    }
    float chosen = 0.0f;
    for (int k = 0; k < top; ++k) {        // the kept groups hold at least `top` outputs, all with finite scores
      int best = 0;
      float bz = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float z = c_s[e];
        if (z > bz) { bz = z; best = e; }
      }
      ids[(size_t)row * top + k] = best;
      weights[(size_t)row * top + k] = z_s[best];
      chosen += z_s[best];
      c_s[best] = -INFINITY;
    }
    const float inv = 1.0f / (chosen + weight_eps);
    for (int k = 0; k < top; ++k) weights[(size_t)row * top + k] *= inv;
  }
}

// out[row] = sum_k w[row, k] * (ids[row, k] < n_real ? Y[pos_of_pair[row, k]] : h[row])   (outputs from n_real on pass
// their input through) + addend_gate[row] * addend[row] (a result every token gets, scaled per token)
template <typename T>
__global__ void moe_combine_weighted_kernel(T* __restrict__ out, const T* __restrict__ Y, int64_t ldy,
                                            const int* __restrict__ pos_of_pair, const int* __restrict__ ids,
                                            const float* __restrict__ pair_w, int n_real, const T* __restrict__ h,
                                            int64_t ldh, int W, int top, const T* __restrict__ addend, int64_t ld_add,
                                            const float* __restrict__ addend_gate) {
  const int row = blockIdx.x;
  const float ag = addend ? (addend_gate ? addend_gate[row] : 1.0f) : 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const size_t p = (size_t)row * top + k;
      const float v = ids[p] < n_real ? Num<T>::to_f(Y[(size_t)pos_of_pair[p] * ldy + i])
                                      : Num<T>::to_f(h[(size_t)row * ldh + i]);
      acc += pair_w[p] * v;
    }
    if (addend) acc += ag * Num<T>::to_f(addend[(size_t)row * ld_add + i]);
    out[(size_t)row * W + i] = Num<T>::from_f(acc);
  }
}

#define MOE_DISPATCH(dtype, ...)                                                 \
  switch (dtype) {                                                               \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case B200_FP16: { using T = __half; __VA_ARGS__; break; }                    \
    case B200_FP32: { using T = float; __VA_ARGS__; break; }                     \
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);      \
  }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_moe_route(int32_t* expert_ids, float* weights, const void* h, int64_t ldh,
                   const float* router_weight, int64_t rows, int64_t W, int64_t E, int64_t top, int dtype,
                   b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(expert_ids && weights && h && router_weight, "moe_route: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && ldh >= W && E >= 1 && E <= kMaxExperts && top >= 1 && top <= E &&
                     top <= kMaxTop,
                 "moe_route: bad shape (experts <= 1024, top <= min(experts, 32))");
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (moe_route_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                          expert_ids, weights, static_cast<const T*>(h), ldh, router_weight, (int)W, (int)E,
                          (int)top)));
  B200_LAUNCH_OK("moe_route_kernel");
  return B200_OK;
}

int b200_moe_plan(int32_t* offsets, int32_t* sorted_pair, int32_t* pos_of_pair, const int32_t* expert_ids,
                  int64_t n_pairs, int64_t E, b200_stream_t stream) {
  B200_CHECK_ARG(offsets && sorted_pair && pos_of_pair && expert_ids, "moe_plan: null pointer");
  B200_CHECK_ARG(n_pairs >= 0 && n_pairs < (1ll << 31) && E >= 1 && E <= kMaxExperts, "moe_plan: bad shape");
  moe_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(offsets, sorted_pair, pos_of_pair,
                                                                    expert_ids, (int)n_pairs, (int)E);
  B200_LAUNCH_OK("moe_plan_kernel");
  return B200_OK;
}

int b200_grouped_gemm(void* C, int64_t ldc, const void* A, int64_t lda, const int32_t* sorted_pair,
                      const float* pair_scale, int64_t top, const void* weights, const int32_t* offsets,
                      int64_t n_rows, int64_t E, int64_t N, int64_t K, int dtype, b200_stream_t stream) {
  if (n_rows == 0) return B200_OK;
  B200_CHECK_ARG(C && A && weights && offsets, "grouped_gemm: null pointer");
  B200_CHECK_ARG(n_rows > 0 && E >= 1 && N > 0 && K > 0 && ldc >= N && lda >= K && top >= 1 &&
                     (n_rows + BM - 1) / BM + E <= 65535,
                 "grouped_gemm: bad shape");
  dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((n_rows + BM - 1) / BM + E));
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (grouped_gemm_kernel<T><<<grid, 256, 0, st>>>(
                          static_cast<T*>(C), ldc, static_cast<const T*>(A), lda, sorted_pair, pair_scale,
                          (int)top, static_cast<const T*>(weights), offsets, (int)E, (int)N, (int)K)));
  B200_LAUNCH_OK("grouped_gemm_kernel");
  return B200_OK;
}

int b200_grouped_gemv(void* C, int64_t ldc, const void* A, int64_t lda, const int32_t* sorted_pair,
                      const float* pair_scale, int64_t top, const void* weights, const int32_t* offsets,
                      int64_t n_rows, int64_t E, int64_t N, int64_t K, int dtype, b200_stream_t stream) {
  if (n_rows == 0) return B200_OK;
  B200_CHECK_ARG(C && A && weights && offsets, "grouped_gemv: null pointer");
  const int es = dtype == B200_FP32 ? 4 : 2;
  B200_CHECK_ARG(E >= 1 && E <= 65535 && N > 0 && K > 0 && ldc >= N && lda >= K && top >= 1 && (K * es) % 16 == 0 &&
                     is_aligned(weights, 16) && (int64_t)GV_MB * K * es <= 200 * 1024,
                 "grouped_gemv: K rows of 16-byte multiples that fit in shared memory %d at a time", GV_MB);
  const size_t smem = (size_t)GV_MB * K * es;
  dim3 grid((unsigned)((N + GV_WARPS * GV_CPW - 1) / (GV_WARPS * GV_CPW)), (unsigned)E);
  auto st = static_cast<cudaStream_t>(stream);
#define GV_LAUNCH(T)                                                                                      \
  {                                                                                                       \
    auto kern = grouped_gemv_kernel<T>;                                                                   \
    if (smem > 48 * 1024)                                                                                 \
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    kern<<<grid, GV_WARPS * 32, smem, st>>>(static_cast<T*>(C), ldc, static_cast<const T*>(A), lda,       \
                                            sorted_pair, pair_scale, (int)top, static_cast<const T*>(weights), \
                                            offsets, (int)N, (int)K);                                     \
  }
  switch (dtype) {
    case B200_BF16: GV_LAUNCH(__nv_bfloat16); break;
    case B200_FP16: GV_LAUNCH(__half); break;
    case B200_FP32: GV_LAUNCH(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef GV_LAUNCH
  B200_LAUNCH_OK("grouped_gemv_kernel");
  return B200_OK;
}

int b200_moe_gather(void* xs, const void* h, int64_t ldh, const int32_t* sorted_pair, const float* pair_scale,
                    int64_t top, int64_t n_pairs, int64_t W, int dtype, b200_stream_t stream) {
  if (n_pairs == 0) return B200_OK;
  B200_CHECK_ARG(xs && h && sorted_pair, "moe_gather: null pointer");
  B200_CHECK_ARG(n_pairs > 0 && W > 0 && ldh >= W && top >= 1, "moe_gather: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (moe_gather_kernel<T><<<(unsigned)n_pairs, 256, 0, st>>>(
                          static_cast<T*>(xs), static_cast<const T*>(h), ldh, sorted_pair, pair_scale, (int)top, (int)W)));
  B200_LAUNCH_OK("moe_gather_kernel");
  return B200_OK;
}

int b200_moe_combine(void* out, const void* Y, int64_t ldy, const int32_t* pos_of_pair, int64_t rows,
                     int64_t W, int64_t top, float scale, const void* addend, int64_t ld_add, int dtype,
                     b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && Y && pos_of_pair, "moe_combine: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && ldy >= W && top >= 1 && (!addend || ld_add >= W), "moe_combine: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (moe_combine_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                          static_cast<T*>(out), static_cast<const T*>(Y), ldy, pos_of_pair, (int)W, (int)top, scale,
                          static_cast<const T*>(addend), ld_add)));
  B200_LAUNCH_OK("moe_combine_kernel");
  return B200_OK;
}

int b200_moe_table_route(int32_t* expert_ids, const int32_t* table, const int32_t* tokens, int64_t rows, int64_t top,
                         int64_t vocab, int64_t E, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(expert_ids && table && tokens, "moe_table_route: null pointer");
  B200_CHECK_ARG(rows > 0 && top >= 1 && top <= kMaxTop && vocab > 0 && E >= 1 && E <= kMaxExperts &&
                     rows * top < (1ll << 31),
                 "moe_table_route: bad shape");
  const int64_t n = rows * top;
  int64_t grid = (n + 255) / 256;
  if (grid > 4096) grid = 4096;
  moe_table_route_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      expert_ids, table, tokens, n, (int)top, (int)vocab, (int)E);
  B200_LAUNCH_OK("moe_table_route_kernel");
  return B200_OK;
}

int b200_moe_route_softmax(int32_t* expert_ids, float* weights, float* extra_out, const void* h, int64_t ldh,
                           const float* router_weight, const float* correction, const float* extra_weight,
                           int64_t rows, int64_t W, int64_t E, int64_t top, int64_t n_groups, int64_t keep_groups,
                           float weight_eps, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(expert_ids && weights && h && router_weight && (!extra_weight || extra_out),
                 "moe_route_softmax: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && ldh >= W && E >= 1 && E <= kMaxExperts && top >= 1 && top <= E &&
                     top <= kMaxTop && n_groups >= 1 && E % n_groups == 0 && keep_groups >= 1 &&
                     keep_groups <= n_groups && top <= keep_groups * (E / n_groups),
                 "moe_route_softmax: bad shape (outputs <= 1024 in equal groups, top <= min(32, outputs of the kept "
                 "groups))");
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (moe_route_softmax_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                          expert_ids, weights, extra_out, static_cast<const T*>(h), ldh, router_weight, correction,
                          extra_weight, (int)W, (int)E, (int)top, (int)n_groups, (int)keep_groups, weight_eps)));
  B200_LAUNCH_OK("moe_route_softmax_kernel");
  return B200_OK;
}

int b200_moe_combine_weighted(void* out, const void* Y, int64_t ldy, const int32_t* pos_of_pair,
                              const int32_t* expert_ids, const float* pair_weights, int64_t n_real, const void* h,
                              int64_t ldh, int64_t rows, int64_t W, int64_t top, const void* addend, int64_t ld_add,
                              const float* addend_gate, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && Y && pos_of_pair && expert_ids && pair_weights && h, "moe_combine_weighted: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && ldy >= W && ldh >= W && top >= 1 && (!addend || ld_add >= W),
                 "moe_combine_weighted: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  MOE_DISPATCH(dtype, (moe_combine_weighted_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                          static_cast<T*>(out), static_cast<const T*>(Y), ldy, pos_of_pair, expert_ids, pair_weights,
                          (int)n_real, static_cast<const T*>(h), ldh, (int)W, (int)top,
                          static_cast<const T*>(addend), ld_add, addend_gate)));
  B200_LAUNCH_OK("moe_combine_weighted_kernel");
  return B200_OK;
}

}  // extern "C"
