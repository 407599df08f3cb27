// delta_rule.cu — generalised delta-rule recurrence with a per-channel decay and removal rate.
//
// Per head, state S [d (key) x d (value)] in fp32, carried per sequence in a state slot:
//     w_t = exp(-decay_scale * sigmoid(wl_t + w0))        decay per key channel
//     a_t = sigmoid(al_t + a0)                            removal rate per key channel
//     u_t = k_t / sqrt(|k_t|^2 + key_eps)                 unit key
//     S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T
//     o_t = S_t^T r_t
//     out = o_t / rms(o_t) * nw * sigmoid(g_t)            per-head RMS, channel weight, output gate
// One CTA per (sequence, head); thread j owns column j of S in registers and walks the step's
// tokens of that sequence in order (a single decoded token or a whole prompt portion).  A portion
// that starts at position 0 starts from S = 0 instead of reading the slot.
#include "common.cuh"

namespace b200 {
namespace {

template <typename T, int DK>
__global__ void __launch_bounds__(DK < 32 ? 32 : DK)
delta_rule_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ r, const T* __restrict__ k,
                  const T* __restrict__ v, const T* __restrict__ wl, const T* __restrict__ al,
                  const T* __restrict__ g, int64_t ld, int64_t ld_w, const float* __restrict__ w0,
                  const float* __restrict__ a0, const float* __restrict__ nw, float* __restrict__ state,
                  const int* __restrict__ q_cu, const int* __restrict__ positions,
                  const int* __restrict__ state_slots, int H, int d, float decay_scale, float key_eps,
                  float eps) {
  constexpr int NT = DK < 32 ? 32 : DK;
  __shared__ __align__(16) float r_s[DK], k_s[DK], u_s[DK], w_s[DK], au_s[DK];
  __shared__ float red[32], red2[32];   // alternate: block_sum does not sync after reading
  const int seq = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int t0 = q_cu[seq], t1 = q_cu[seq + 1];
  if (t0 >= t1) return;
  const bool live = j < d;
  if (j < DK && !live) r_s[j] = k_s[j] = u_s[j] = w_s[j] = au_s[j] = 0.0f;   // padding entries stay zero
  float* Sg = state + (((size_t)state_slots[seq] * H + h) * d) * d;   // [key][value]
  float S[DK];
  const bool fresh = positions[t0] == 0;
#pragma unroll
  for (int kk = 0; kk < DK; ++kk) S[kk] = (live && kk < d && !fresh) ? Sg[(size_t)kk * d + j] : 0.0f;
  const int c = h * d + j;
  const float w0j = live ? w0[c] : 0.0f, a0j = live ? a0[c] : 0.0f, nwj = live ? nw[c] : 0.0f;
  // the six inputs of token t + 1 are loaded while token t is computed: the recurrence itself is short,
  // a dependent global load per token would dominate it
  float nk = 0.0f, nv = 0.0f, nr = 0.0f, nwl = 0.0f, nal = 0.0f, ng = 0.0f;
  auto load_token = [&](int t) {
    if (live) {
      const size_t base = (size_t)t * ld + c;
      nk = Num<T>::to_f(k[base]);
      nv = Num<T>::to_f(v[base]);
      nr = Num<T>::to_f(r[base]);
      nal = Num<T>::to_f(al[base]);
      ng = Num<T>::to_f(g[base]);
      nwl = Num<T>::to_f(wl[(size_t)t * ld_w + c]);
    }
  };
  load_token(t0);
  for (int t = t0; t < t1; ++t) {
    const float kj = nk, vj = nv, alj = nal, gj = ng;
    if (live) {
      r_s[j] = nr;
      k_s[j] = kj;
      const float sw = 1.0f / (1.0f + expf(-(nwl + w0j)));
      w_s[j] = expf(-decay_scale * sw);
    }
    if (t + 1 < t1) load_token(t + 1);
    const float k2 = block_sum<NT>(kj * kj, red);   // syncs: the vectors above are visible after it
    if (live) {
      const float uj = kj * rsqrtf(k2 + key_eps);
      const float aj = 1.0f / (1.0f + expf(-(alj + a0j)));
      u_s[j] = uj;
      au_s[j] = aj * uj;
    }
    __syncthreads();
    // both passes over the key dimension read the shared vectors four at a time and keep four partial sums, so
    // that neither the shared-memory loads nor one long chain of dependent FMAs set the pace (entries >= d are 0)
    float us4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 u4 = *reinterpret_cast<const float4*>(u_s + kk);
      us4[0] += u4.x * S[kk]; us4[1] += u4.y * S[kk + 1]; us4[2] += u4.z * S[kk + 2]; us4[3] += u4.w * S[kk + 3];
    }
    const float uS = (us4[0] + us4[1]) + (us4[2] + us4[3]);
    float o4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(w_s + kk);
      const float4 a4 = *reinterpret_cast<const float4*>(au_s + kk);
      const float4 k4 = *reinterpret_cast<const float4*>(k_s + kk);
      const float4 r4 = *reinterpret_cast<const float4*>(r_s + kk);
      S[kk] = w4.x * S[kk] - a4.x * uS + k4.x * vj;             o4[0] += S[kk] * r4.x;
      S[kk + 1] = w4.y * S[kk + 1] - a4.y * uS + k4.y * vj;     o4[1] += S[kk + 1] * r4.y;
      S[kk + 2] = w4.z * S[kk + 2] - a4.z * uS + k4.z * vj;     o4[2] += S[kk + 2] * r4.z;
      S[kk + 3] = w4.w * S[kk + 3] - a4.w * uS + k4.w * vj;     o4[3] += S[kk + 3] * r4.w;
    }
    const float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    const float o2 = block_sum<NT>(live ? o * o : 0.0f, red2);   // also fences the smem vectors
    if (live) {
      const float gate = 1.0f / (1.0f + expf(-gj));
      out[(size_t)t * ldo + c] = Num<T>::from_f(o * rsqrtf(o2 / (float)d + eps) * nwj * gate);
    }
  }
  if (live) {
#pragma unroll
    for (int kk = 0; kk < DK; ++kk)
      if (kk < d) Sg[(size_t)kk * d + j] = S[kk];
  }
}

template <typename T>
int launch_delta(void* out, int64_t ldo, const void* r, const void* k, const void* v, const void* wl,
                 const void* al, const void* g, int64_t ld, int64_t ld_w, const float* w0, const float* a0,
                 const float* nw, float* state, const int* q_cu, const int* positions,
                 const int* state_slots, int64_t n_seq, int H, int d, float decay_scale, float key_eps,
                 float eps, cudaStream_t st) {
  dim3 grid((unsigned)n_seq, (unsigned)H);
#define DR_LAUNCH(DK)                                                                                 \
  delta_rule_kernel<T, DK><<<grid, (DK < 32 ? 32 : DK), 0, st>>>(                                      \
      static_cast<T*>(out), ldo, static_cast<const T*>(r), static_cast<const T*>(k),                   \
      static_cast<const T*>(v), static_cast<const T*>(wl), static_cast<const T*>(al),                  \
      static_cast<const T*>(g), ld, ld_w, w0, a0, nw, state, q_cu, positions, state_slots, H, d, decay_scale, \
      key_eps, eps)
  if (d <= 32) DR_LAUNCH(32);
  else if (d <= 64) DR_LAUNCH(64);
  else if (d <= 128) DR_LAUNCH(128);
  else return set_error(B200_ERR_UNSUPPORTED, "delta_rule: head size %d > 128", d);
#undef DR_LAUNCH
  B200_LAUNCH_OK("delta_rule_kernel");
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_delta_rule(void* out, int64_t ldo, const void* r, const void* k, const void* v,
                    const void* decay_logits, const void* removal_logits, const void* gate_logits,
                    int64_t ld, int64_t ld_decay, const float* decay_bias, const float* removal_bias,
                    const float* norm_weight, float* state, const int32_t* q_cu_lens,
                    const int32_t* positions, const int32_t* state_slots, int64_t n_seq, int64_t H,
                    int64_t d, float decay_scale, float key_eps, float eps, int dtype,
                    b200_stream_t stream) {
  if (n_seq == 0) return B200_OK;
  B200_CHECK_ARG(out && r && k && v && decay_logits && removal_logits && gate_logits && decay_bias &&
                     removal_bias && norm_weight && state && q_cu_lens && positions && state_slots,
                 "delta_rule: null pointer");
  B200_CHECK_ARG(n_seq > 0 && H > 0 && H <= 65535 && d > 0 && ldo >= H * d && ld >= H * d && ld_decay >= H * d, "delta_rule: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define DR_CALL(T)                                                                                      \
  return launch_delta<T>(out, ldo, r, k, v, decay_logits, removal_logits, gate_logits, ld, ld_decay, decay_bias,  \
                         removal_bias, norm_weight, state, q_cu_lens, positions, state_slots, n_seq,    \
                         (int)H, (int)d, decay_scale, key_eps, eps, st)
  switch (dtype) {
    case B200_BF16: DR_CALL(__nv_bfloat16);
    case B200_FP16: DR_CALL(__half);
    case B200_FP32: DR_CALL(float);
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef DR_CALL
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Gated delta rule with a decay per key channel and short causal filters on its inputs.
//
// Per head, state S [dim (key) x vdim (value)] in fp32, carried per sequence in a state slot:
//     x      = silu(filter(W h))            per channel: y_t = sum_i c[i] x_{t - (taps - 1) + i}, zeros before the start
//     q, k   = x / sqrt(|x|^2 + unit_eps)   per head; q also times dim^(-1/2)
//     d_t    = exp(-exp(A_h) softplus(a_t + dt))              decay per head and key channel
//     b_t    = sigmoid(beta logit)                            per head
//     S <- diag(d_t) S ;  u = b_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//     out    = o_t / rms(o_t) * nw * sigmoid(g_t)             per-head RMS, channel weight [vdim], output gate
// Value head h reads query/key head h / (H / G).
//
//   prepare : every row in parallel: filters (the lags that reach before the step come from the sequence's filter
//             state [slot, taps - 1, channels]), silu, unit length, decay and beta -> fp32 rows
//   carry   : the filter state takes the last taps - 1 inputs of every sequence (after prepare has read it)
//   scan    : one CTA per (sequence, head); thread j owns column j of S in registers and walks the sequence's rows of
//             the step in order.  A portion that starts at position 0 starts from S = 0 instead of reading the slot.
namespace b200 {
namespace {

constexpr int kGdPrepThreads = 128;
constexpr int kMaxTaps = 16;

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// filtered input of channel c (of `n_ch` in a [q | k | v] row) for the row `row`, in-step index r, position pos
template <typename T>
__device__ __forceinline__ float filtered(const T* __restrict__ x, int64_t ld, const float* __restrict__ w,
                                          const float* __restrict__ fstate, int n_state_ch, int state_c, int row,
                                          int r, int pos, int c, int taps) {
  float acc = 0.0f;
  for (int lag = 0; lag < taps; ++lag) {
    if (pos - lag < 0) break;                                       // before the start of the sequence: zero
    float v;
    if (r - lag >= 0) v = Num<T>::to_f(x[(size_t)(row - lag) * ld + c]);
    else v = fstate[(size_t)(taps - 1 + r - lag) * n_state_ch + state_c];
    acc += w[(size_t)c * taps + (taps - 1 - lag)] * v;
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(kGdPrepThreads)
gated_delta_prepare_kernel(float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                           float* __restrict__ decay_out, float* __restrict__ beta_out, const T* __restrict__ q_in,
                           const T* __restrict__ k_in, const T* __restrict__ v_in, const T* __restrict__ beta_in,
                           int64_t ld, const T* __restrict__ a_in, int64_t ld_a, const float* __restrict__ wq,
                           const float* __restrict__ wk, const float* __restrict__ wv,
                           const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                           const float* __restrict__ fstate, const int* __restrict__ q_cu,
                           const int* __restrict__ positions, const int* __restrict__ token_seq,
                           const int* __restrict__ state_slots, int H, int G, int dim, int vdim, int taps,
                           float unit_eps) {
  // a row's work is shared out over gridDim.y CTAs (steps of few rows would otherwise leave most SMs idle)
  const int row = blockIdx.x, lane = threadIdx.x & 31;
  const int warp = blockIdx.y * (kGdPrepThreads / 32) + (threadIdx.x >> 5), n_warps = gridDim.y * (kGdPrepThreads / 32);
  const int tid = blockIdx.y * kGdPrepThreads + threadIdx.x, n_thr = gridDim.y * kGdPrepThreads;
  const int seq = token_seq[row], r = row - q_cu[seq], pos = positions[row];
  const int nqk = G * dim, nv = H * vdim, n_ch = 2 * nqk + nv;
  const float* fs = fstate + (size_t)state_slots[seq] * (taps - 1) * n_ch;
  // queries and keys: a warp per head, the head's filtered channels stay in registers for the unit norm
  for (int u = warp; u < 2 * G; u += n_warps) {
    const bool is_q = u < G;
    const int head = is_q ? u : u - G;
    const T* x = is_q ? q_in : k_in;
    const float* w = is_q ? wq : wk;
    float vals[8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = lane + 32 * i;
      vals[i] = 0.0f;
      if (t < dim) {
        const int c = head * dim + t;
        vals[i] = silu_f(filtered<T>(x, ld, w, fs, n_ch, (is_q ? 0 : nqk) + c, row, r, pos, c, taps));
        ss += vals[i] * vals[i];
      }
    }
    ss = warp_sum(ss);
    const float sc = (is_q ? rsqrtf((float)dim) : 1.0f) / sqrtf(ss + unit_eps);
    float* dst = (is_q ? q_out : k_out) + (size_t)row * nqk + (size_t)head * dim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = lane + 32 * i;
      if (t < dim) dst[t] = vals[i] * sc;
    }
  }
  for (int c = tid; c < nv; c += n_thr)
    v_out[(size_t)row * nv + c] = silu_f(filtered<T>(v_in, ld, wv, fs, n_ch, 2 * nqk + c, row, r, pos, c, taps));
  for (int c = tid; c < H * dim; c += n_thr) {
    const float sp = softplus_f(Num<T>::to_f(a_in[(size_t)row * ld_a + c]) + dt_bias[c]);
    decay_out[(size_t)row * H * dim + c] = expf(-expf(a_log[c / dim]) * sp);
  }
  for (int h = tid; h < H; h += n_thr)
    beta_out[(size_t)row * H + h] = 1.0f / (1.0f + expf(-Num<T>::to_f(beta_in[(size_t)row * ld + h])));
}

// fstate[slot, i] <- the input at in-step index n - (taps - 1) + i, or the old entry i + n where that is before the step
template <typename T>
__global__ void filter_state_carry_kernel(float* __restrict__ fstate, const T* __restrict__ q_in,
                                          const T* __restrict__ k_in, const T* __restrict__ v_in, int64_t ld,
                                          const int* __restrict__ q_cu, const int* __restrict__ state_slots,
                                          int nqk, int nv, int taps) {
  const int seq = blockIdx.x;
  const int t0 = q_cu[seq], n = q_cu[seq + 1] - t0;
  if (n <= 0) return;
  const int n_ch = 2 * nqk + nv;
  float* fs = fstate + (size_t)state_slots[seq] * (taps - 1) * n_ch;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n_ch; c += gridDim.y * blockDim.x) {
    const T* x = c < nqk ? q_in + c : (c < 2 * nqk ? k_in + (c - nqk) : v_in + (c - 2 * nqk));
    for (int i = 0; i < taps - 1; ++i) {            // ascending: entry i reads entry i + n > i of the old state
      const int r = n - (taps - 1) + i;
      fs[(size_t)i * n_ch + c] = r >= 0 ? Num<T>::to_f(x[(size_t)(t0 + r) * ld]) : fs[(size_t)(i + n) * n_ch + c];
    }
  }
}

// KS threads share a column of S: thread (column c, part) keeps the DK / KS key rows [part * DK / KS, ...) of the
// column, and the two sums over the key dimension end in a butterfly over the KS neighbouring lanes.  KS = 1 is the
// form for key sizes up to 128 (at 128 x 128 two threads per column measured 1.3x slower: the spills and the wider
// barriers cost more than the shorter serial work saves); KS = 2 carries key sizes up to 256, whose columns do not
// fit one thread's registers.
template <typename T, int DK, int NT, int KS>
__global__ void __launch_bounds__(NT)
gated_delta_scan_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const float* __restrict__ k,
                        const float* __restrict__ v, const float* __restrict__ decay, const float* __restrict__ beta,
                        const T* __restrict__ gate, int64_t ld_gate, const float* __restrict__ nw,
                        float* __restrict__ state, const int* __restrict__ q_cu, const int* __restrict__ positions,
                        const int* __restrict__ state_slots, int H, int G, int dim, int vdim, float eps,
                        float* __restrict__ raw) {
  // raw != nullptr: the read-outs leave as they are (fp32 [rows, H * vdim]) and a token-parallel launch applies the
  // norm and the gate afterwards, so that the walk has one barrier per token instead of two and no reduction
  constexpr int DL = DK / KS;                       // key rows a thread keeps
  __shared__ __align__(16) float q_s[2][DK], k_s[2][DK], w_s[2][DK];
  __shared__ float red[32];
  const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int j = tid / KS, part = tid % KS, k0 = part * DL;
  const int t0 = q_cu[seq], t1 = q_cu[seq + 1];
  if (t0 >= t1) return;
  const int g = h / (H / G);
  const bool live = j < vdim;
  const int nqk = G * dim, nv = H * vdim, nd = H * dim;
  float* Sg = state + (((size_t)state_slots[seq] * H + h) * dim) * vdim;   // [key][value]
  float S[DL];
  const bool fresh = positions[t0] == 0;
#pragma unroll
  for (int kk = 0; kk < DL; ++kk) S[kk] = (live && k0 + kk < dim && !fresh) ? Sg[(size_t)(k0 + kk) * vdim + j] : 0.0f;
  for (int kk = tid; kk < DK; kk += NT)
    if (kk >= dim) q_s[0][kk] = q_s[1][kk] = k_s[0][kk] = k_s[1][kk] = w_s[0][kk] = w_s[1][kk] = 0.0f;
  const float nwj = live ? nw[j] : 0.0f;
  constexpr int PER = (DK + NT - 1) / NT;        // key channels a thread stages per token
  float nq[PER], nk[PER], nd_[PER], nvj = 0.0f, nb = 0.0f, ng = 0.0f;
  auto load_token = [&](int t) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int kk = tid + i * NT;
      if (kk < dim) {
        nq[i] = q[(size_t)t * nqk + (size_t)g * dim + kk];
        nk[i] = k[(size_t)t * nqk + (size_t)g * dim + kk];
        nd_[i] = decay[(size_t)t * nd + (size_t)h * dim + kk];
      }
    }
    nb = beta[(size_t)t * H + h];
    if (live) {
      nvj = v[(size_t)t * nv + (size_t)h * vdim + j];
      ng = Num<T>::to_f(gate[(size_t)t * ld_gate + (size_t)h * vdim + j]);
    }
  };
  load_token(t0);
  for (int t = t0; t < t1; ++t) {
    const int b = (t - t0) & 1;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int kk = tid + i * NT;
      if (kk < dim) { q_s[b][kk] = nq[i]; k_s[b][kk] = nk[i]; w_s[b][kk] = nd_[i]; }
    }
    const float vj = nvj, bt = nb, gj = ng;
    if (t + 1 < t1) load_token(t + 1);       // the next token's inputs arrive while this one is computed
    __syncthreads();
    float ks4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DL; kk += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(&w_s[b][k0 + kk]);
      const float4 k4 = *reinterpret_cast<const float4*>(&k_s[b][k0 + kk]);
      S[kk] *= w4.x;     ks4[0] += k4.x * S[kk];
      S[kk + 1] *= w4.y; ks4[1] += k4.y * S[kk + 1];
      S[kk + 2] *= w4.z; ks4[2] += k4.z * S[kk + 2];
      S[kk + 3] *= w4.w; ks4[3] += k4.w * S[kk + 3];
    }
    float kS = (ks4[0] + ks4[1]) + (ks4[2] + ks4[3]);
#pragma unroll
    for (int sh = KS / 2; sh > 0; sh >>= 1) kS += __shfl_xor_sync(0xffffffffu, kS, sh);
    const float u = bt * (vj - kS);
    float o4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DL; kk += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(&k_s[b][k0 + kk]);
      const float4 q4 = *reinterpret_cast<const float4*>(&q_s[b][k0 + kk]);
      S[kk] += k4.x * u;     o4[0] += S[kk] * q4.x;
      S[kk + 1] += k4.y * u; o4[1] += S[kk + 1] * q4.y;
      S[kk + 2] += k4.z * u; o4[2] += S[kk + 2] * q4.z;
      S[kk + 3] += k4.w * u; o4[3] += S[kk + 3] * q4.w;
    }
    float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
#pragma unroll
    for (int sh = KS / 2; sh > 0; sh >>= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
    if (!live) o = 0.0f;
    if (raw) {              // (the barrier of the next token orders this token's reads before the token after next
                            // overwrites the same staging buffer)
      if (live && part == 0) raw[(size_t)t * nv + (size_t)h * vdim + j] = o;
      continue;
    }
    const float o2 = block_sum<NT>(part == 0 ? o * o : 0.0f, red);   // its barrier also orders this token's reads
                                                                     // before the token after next overwrites the
                                                                     // same staging buffer
    if (live && part == 0) {
      const float gt = 1.0f / (1.0f + expf(-gj));
      out[(size_t)t * ldo + (size_t)h * vdim + j] = Num<T>::from_f(o * rsqrtf(o2 / (float)vdim + eps) * nwj * gt);
    }
  }
  if (live) {
#pragma unroll
    for (int kk = 0; kk < DL; ++kk)
      if (k0 + kk < dim) Sg[(size_t)(k0 + kk) * vdim + j] = S[kk];
  }
}

// out[row, h] = raw / rms(raw) * nw * sigmoid(gate): a warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ raw, const T* __restrict__ gate,
                      int64_t ld_gate, const float* __restrict__ nw, int64_t n_units, int H, int vdim, float eps) {
  const int64_t u = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (u >= n_units) return;
  const int64_t row = u / H;
  const int h = (int)(u - row * H);
  const float* r = raw + (size_t)u * vdim;
  float ss = 0.0f;
  for (int i = lane; i < vdim; i += 32) ss += r[i] * r[i];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    const float gt = 1.0f / (1.0f + expf(-Num<T>::to_f(gate[(size_t)row * ld_gate + (size_t)h * vdim + i])));
    out[(size_t)row * ldo + (size_t)h * vdim + i] = Num<T>::from_f(r[i] * inv * nw[i] * gt);
  }
}

#define GD_DISPATCH(dtype, ...)                                                  \
  switch (dtype) {                                                               \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case B200_FP16: { using T = __half; __VA_ARGS__; break; }                    \
    case B200_FP32: { using T = float; __VA_ARGS__; break; }                     \
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);      \
  }

template <typename T, int DK>
int launch_gd_scan(int nt, dim3 grid, cudaStream_t st, void* out, int64_t ldo, const float* q, const float* k,
                   const float* v, const float* decay, const float* beta, const void* gate, int64_t ld_gate,
                   const float* nw, float* state, const int* q_cu, const int* positions, const int* slots, int H,
                   int G, int dim, int vdim, float eps, float* raw, int64_t rows) {
#define GD_NT(N, KSP)                                                                                              \
  gated_delta_scan_kernel<T, DK, N, KSP><<<grid, N, 0, st>>>(static_cast<T*>(out), ldo, q, k, v, decay, beta,        \
                                                             static_cast<const T*>(gate), ld_gate, nw, state, q_cu, \
                                                             positions, slots, H, G, dim, vdim, eps, raw)
  if constexpr (DK > 128) {          // two threads per column: value sizes up to 128
    if (nt <= 32) GD_NT(64, 2);
    else if (nt <= 64) GD_NT(128, 2);
    else if (nt <= 128) GD_NT(256, 2);
    else return set_error(B200_ERR_UNSUPPORTED, "gated_delta_scan: key size above 128 with value size above 128");
  } else {
    if (nt <= 32) GD_NT(32, 1);
    else if (nt <= 64) GD_NT(64, 1);
    else if (nt <= 128) GD_NT(128, 1);
    else GD_NT(256, 1);
  }
#undef GD_NT
  B200_LAUNCH_OK("gated_delta_scan_kernel");
  if (raw) {
    const int64_t n_units = rows * H;
    head_norm_gate_kernel<T><<<(unsigned)((n_units + 7) / 8), 256, 0, st>>>(
        static_cast<T*>(out), ldo, raw, static_cast<const T*>(gate), ld_gate, nw, n_units, H, vdim, eps);
    B200_LAUNCH_OK("head_norm_gate_kernel");
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_gated_delta_prepare(float* q_out, float* k_out, float* v_out, float* decay_out, float* beta_out,
                             const void* q_in, const void* k_in, const void* v_in, const void* beta_in, int64_t ld,
                             const void* decay_in, int64_t ld_decay, const float* q_filter, const float* k_filter,
                             const float* v_filter, const float* a_log, const float* dt_bias, float* filter_state,
                             const int32_t* q_cu_lens, const int32_t* positions, const int32_t* token_seq,
                             const int32_t* state_slots, int64_t rows, int64_t n_seq, int64_t H, int64_t G,
                             int64_t dim, int64_t vdim, int64_t taps, float unit_eps, int dtype,
                             b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q_out && k_out && v_out && decay_out && beta_out && q_in && k_in && v_in && beta_in && decay_in &&
                     q_filter && k_filter && v_filter && a_log && dt_bias && (filter_state || taps == 1) && q_cu_lens &&
                     positions && token_seq && state_slots,
                 "gated_delta_prepare: null pointer");
  B200_CHECK_ARG(rows > 0 && n_seq > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && dim <= 256 && vdim > 0 &&
                     taps >= 1 && taps <= kMaxTaps,
                 "gated_delta_prepare: bad shape (key size <= 256, taps <= 16, heads a multiple of query/key heads)");
  auto st = static_cast<cudaStream_t>(stream);
  GD_DISPATCH(dtype, {
    // few rows: up to 8 CTAs per row, so that a step of single tokens still fills the SMs
    const int work = (int)((2 * G * dim + H * vdim + H * dim + kGdPrepThreads * 4 - 1) / (kGdPrepThreads * 4));
    int split = (int)((2 * sm_count() + rows - 1) / rows);
    split = split < 1 ? 1 : (split > 8 ? 8 : split);
    if (split > work) split = work < 1 ? 1 : work;
    gated_delta_prepare_kernel<T><<<dim3((unsigned)rows, (unsigned)split), kGdPrepThreads, 0, st>>>(
        q_out, k_out, v_out, decay_out, beta_out, static_cast<const T*>(q_in), static_cast<const T*>(k_in),
        static_cast<const T*>(v_in), static_cast<const T*>(beta_in), ld, static_cast<const T*>(decay_in), ld_decay,
        q_filter, k_filter, v_filter, a_log, dt_bias, filter_state, q_cu_lens, positions, token_seq, state_slots,
        (int)H, (int)G, (int)dim, (int)vdim, (int)taps, unit_eps);
    B200_LAUNCH_OK("gated_delta_prepare_kernel");
    if (taps > 1) {
      const int csplit = (int)((2 * G * dim + H * vdim + 1023) / 1024);
      filter_state_carry_kernel<T><<<dim3((unsigned)n_seq, (unsigned)(csplit > 8 ? 8 : csplit)), 256, 0, st>>>(
          filter_state, static_cast<const T*>(q_in), static_cast<const T*>(k_in), static_cast<const T*>(v_in), ld,
          q_cu_lens, state_slots, (int)(G * dim), (int)(H * vdim), (int)taps);
      B200_LAUNCH_OK("filter_state_carry_kernel");
    }
  });
  return B200_OK;
}

int b200_gated_delta_scan(void* out, int64_t ldo, const float* q, const float* k, const float* v, const float* decay,
                          const float* beta, const void* gate_logits, int64_t ld_gate, const float* norm_weight,
                          float* state, const int32_t* q_cu_lens, const int32_t* positions,
                          const int32_t* state_slots, int64_t n_seq, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                          float eps, float* raw_workspace, int64_t rows, int dtype, b200_stream_t stream) {
  if (n_seq == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k && v && decay && beta && gate_logits && norm_weight && state && q_cu_lens &&
                     positions && state_slots,
                 "gated_delta_scan: null pointer");
  B200_CHECK_ARG(n_seq > 0 && H > 0 && H <= 65535 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 256 &&
                     ldo >= H * vdim && ld_gate >= H * vdim,
                 "gated_delta_scan: bad shape (value size <= 256)");
  auto st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)n_seq, (unsigned)H);
  const int nt = (int)((vdim + 31) / 32 * 32);
#define GD_CALL(DK)                                                                                                  \
  GD_DISPATCH(dtype, return (launch_gd_scan<T, DK>(nt, grid, st, out, ldo, q, k, v, decay, beta, gate_logits, ld_gate, \
                                                   norm_weight, state, q_cu_lens, positions, state_slots, (int)H,     \
                                                   (int)G, (int)dim, (int)vdim, eps, raw_workspace, rows)))
  if (dim <= 32) { GD_CALL(32); }
  else if (dim <= 64) { GD_CALL(64); }
  else if (dim <= 128) { GD_CALL(128); }
  else if (dim <= 256) { GD_CALL(256); }
  else return b200::set_error(B200_ERR_UNSUPPORTED, "gated_delta_scan: key size %d > 256", (int)dim);
#undef GD_CALL
  return B200_OK;
}

}  // extern "C"
