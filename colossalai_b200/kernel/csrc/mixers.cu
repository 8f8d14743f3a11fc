// Sequence-mixer kernels for hybrid decoders on sm_100a: recurrent (linear-attention / delta-rule) layers with a fixed-size
// fp32 state per sequence, short causal convolutions with a carried window, and paged attention with a learned
// distance-bucket bias and an optional softmax sink.  All of them work on a RAGGED step: the flat token batch holds, for
// every live sequence, the next `q_len` tokens (a whole prompt, a portion of one, or one decoded token), described by
//
//   cu_q[nseq + 1]   first flat token index of every sequence's portion
//   ctx_len[nseq]    tokens of the sequence that earlier steps already consumed (0 = a fresh sequence: the carried state
//                    is taken as zero, so a recycled slot needs no clearing)
//   slots[nseq]      index of the sequence's state slot in the per-layer state pool
//
// Every recurrence runs token by token in fp32 with one fixed order of operations, so the result at a position does not
// depend on how the prompt was cut or on what else is in the batch.
//
//   cb_short_conv_silu      y = silu(causal depthwise conv(x) + bias) over time (activation and bias optional), window
//                           of taps-1 inputs carried per slot
//   cb_state_scan           (prepare + scan) per head a matrix M [dim, vdim]: M <- a_h M + outer(k, v) with one decay
//                           per head; or the gated delta rule M <- diag(r) M; e = w (v - M^T k); M <- M + outer(k, e)
//                           with a decay per key channel; or M <- g_t M + w_t outer(k, v) with a decay g_t and a write
//                           strength w_t per token and head (selective state space: from the step size; matrix memory
//                           with exponential gates: from a running maximum, with a normaliser vector beside M); the
//                           read-out y = M^T q follows the write
//   cb_lru_scan             per channel S <- a_t S + sqrt(1 - a_t^2) i_t u_t with gates from fp32 pre-activations
//   cb_gated_group_rmsnorm  out = o / rms_group(o) * w * sigmoid(gate) (or silu(gate); w optional; gate before or
//                           after the norm)
//   cb_rotary_unit_norm     q / k heads in place: rotary positions on a part of the head (half or interleaved pairs),
//                           then division by the head's root mean square
//   cb_norm_mean            mean of up to four RMS-normed [T, W] tensors, fp32 out
//   cb_sigmoid_gate_mul     o *= sigmoid(gate)
//   cb_stream_add_norm      x(fp32) += sum of up to four [T, W] addends + a [W] row;  h = cast(rms / layer norm of x)
//   cb_rotary_half          rotate-half rotary positions from an fp32 [positions, dims] cos|sin table, strided in / out
//   cb_latent_kv_write      latent attention's cache row: [rms_norm(latent) * w | rotated shared key part]
//   cb_clamped_glu          g = min(gate, L); u = clamp(up, -L, L); out = g * sigmoid(alpha g) * (u + 1)
//   cb_rmsnorm_residual     x(fp32) += mult * y / rms(y) * (offset + w);  h = cast(x)
//   cb_rmsnorm_f32in        out = cast(x / rms(x) * (offset + w)) for an fp32 residual stream
//   cb_paged_kv_write_mix   K / V rows (different widths allowed) into the paged cache, V optionally blended with another
//                           layer's values first
//   cb_paged_bias_attention causal attention of every step token over its sequence's paged cache with
//                           score = scale * q.k + table[bucket(distance)][head] - slope[head] * distance, an optional
//                           sink (score 0 or learned per head) in the denominator, a block mask or a sliding window
//   cb_depth_mix            weighted sum over the history of the fp32 stream (+ compute-dtype copy)
//   cb_poly_norm            a N(z) + b N(z^2) + c N(z^3) + e with N = division by the row's root mean square
//   cb_head_rmsnorm         RMS norm per head with a weight over the head's channels (query heads | key heads); optionally
//                           the normed key heads go straight into the paged key cache and the un-normed ones into the
//                           value cache
#include "common.cuh"

namespace {

CB_DEVICE float silu_f(float x) { return x / (1.f + expf(-x)); }
CB_DEVICE float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
CB_DEVICE float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
CB_DEVICE float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
CB_DEVICE float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------------------------------------ short convolution
// The convolution's activation is stored in the compute dtype: for 16-bit outputs the hardware exponential and
// reciprocal (relative error ~1e-6) are far inside the rounding of the store; fp32 keeps the IEEE forms.
template <typename T> CB_DEVICE float conv_silu(float x) { return x * __frcp_rn(1.f + __expf(-x)); }
template <> CB_DEVICE float conv_silu<float>(float x) { return silu_f(x); }

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_TOK_TILE = 32;

template <typename T>
__global__ void __launch_bounds__(128) short_conv_silu_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                              const T* __restrict__ bias,
                                                              const T* __restrict__ state, T* __restrict__ out,
                                                              int64_t ldo, const int* __restrict__ cu_q,
                                                              const int* __restrict__ ctx_len,
                                                              const int* __restrict__ slots, int C, int taps,
                                                              int apply_silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.z;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  const int j0 = blockIdx.y * CONV_TOK_TILE;
  if (c >= C || j0 >= qlen) return;
  const bool carried = ctx_len[s] > 0;
  const T* st = state + (int64_t)slots[s] * (taps - 1) * C;
  float wt[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    wt[i] = i < taps ? to_f32<T>(w[(int64_t)c * taps + i]) : 0.f;
    win[i] = 0.f;
    if (i < taps - 1) {
      const int rel = j0 - (taps - 1) + i;
      if (rel >= 0) win[i] = to_f32<T>(x[(int64_t)(t0 + rel) * ldx + c]);
      else if (carried) win[i] = to_f32<T>(st[(int64_t)(taps - 1 + rel) * C + c]);
    }
  }
  const int j1 = min(j0 + CONV_TOK_TILE, qlen);
  const float bv = bias != nullptr ? to_f32<T>(bias[c]) : 0.f;
  for (int j = j0; j < j1; ++j) {
    const float cur = to_f32<T>(x[(int64_t)(t0 + j) * ldx + c]);
    float acc = bv;
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
      if (i < taps - 1) acc = fmaf(wt[i], win[i], acc);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i)
      if (i == taps - 1) acc = fmaf(wt[i], cur, acc);
    out[(int64_t)(t0 + j) * ldo + c] = from_f32<T>(apply_silu ? conv_silu<T>(acc) : acc);
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
      if (i < taps - 2) win[i] = win[i + 1];
      else if (i == taps - 2) win[i] = cur;
    }
  }
}

// 16 bytes of adjacent channels per thread (8 x 16-bit or 4 x fp32) for up to 4 taps: the row segment a warp touches is
// 512 bytes instead of 64.  Needs channel count, row strides and base addresses that are multiples of the vector.
constexpr int CONV_VEC_TAPS = 4;

template <typename T>
__global__ void __launch_bounds__(128) short_conv_silu_vec_kernel(const T* __restrict__ x, int64_t ldx,
                                                                  const T* __restrict__ w, const T* __restrict__ bias,
                                                                  const T* __restrict__ state,
                                                                  T* __restrict__ out, int64_t ldo,
                                                                  const int* __restrict__ cu_q,
                                                                  const int* __restrict__ ctx_len,
                                                                  const int* __restrict__ slots, int C, int taps,
                                                                  int apply_silu) {
  constexpr int V = Vec16<T>::N;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  const int s = blockIdx.z;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  const int j0 = blockIdx.y * CONV_TOK_TILE;
  if (c >= C || j0 >= qlen) return;
  const bool carried = ctx_len[s] > 0;
  const T* st = state + (int64_t)slots[s] * (taps - 1) * C;
  float wt[CONV_VEC_TAPS][V], win[CONV_VEC_TAPS - 1][V], bv[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    bv[e] = bias != nullptr ? to_f32<T>(bias[c + e]) : 0.f;
#pragma unroll
    for (int i = 0; i < CONV_VEC_TAPS; ++i) wt[i][e] = i < taps ? to_f32<T>(w[(int64_t)(c + e) * taps + i]) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < CONV_VEC_TAPS - 1; ++i) {
    Vec16<T> v;
    v.raw = make_uint4(0u, 0u, 0u, 0u);
    if (i < taps - 1) {
      const int rel = j0 - (taps - 1) + i;
      if (rel >= 0) v.load(x + (int64_t)(t0 + rel) * ldx + c);
      else if (carried) v.load(st + (int64_t)(taps - 1 + rel) * C + c);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) win[i][e] = v.get(e);
  }
  const int j1 = min(j0 + CONV_TOK_TILE, qlen);
  for (int j = j0; j < j1; ++j) {
    Vec16<T> v, o;
    v.load(x + (int64_t)(t0 + j) * ldx + c);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float cur = v.get(e);
      float acc = bv[e];
#pragma unroll
      for (int i = 0; i < CONV_VEC_TAPS - 1; ++i)
        if (i < taps - 1) acc = fmaf(wt[i][e], win[i][e], acc);
#pragma unroll
      for (int i = 0; i < CONV_VEC_TAPS; ++i)
        if (i == taps - 1) acc = fmaf(wt[i][e], cur, acc);
      o.set(e, apply_silu ? conv_silu<T>(acc) : acc);
#pragma unroll
      for (int i = 0; i < CONV_VEC_TAPS - 1; ++i) {
        if (i < taps - 2) win[i][e] = win[i + 1][e];
        else if (i == taps - 2) win[i][e] = cur;
      }
    }
    o.store(out + (int64_t)(t0 + j) * ldo + c);
  }
}

// the window a later step starts from: the last taps-1 inputs of the sequence (older ones come from the old window
// when the portion is shorter than that); every thread reads all it needs before it writes
template <typename T>
__global__ void __launch_bounds__(128) short_conv_state_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ state,
                                                               const int* __restrict__ cu_q,
                                                               const int* __restrict__ ctx_len,
                                                               const int* __restrict__ slots, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  if (c >= C || qlen == 0) return;
  const bool carried = ctx_len[s] > 0;
  T* st = state + (int64_t)slots[s] * (taps - 1) * C;
  T val[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
    val[i] = from_f32<T>(0.f);
    if (i < taps - 1) {
      const int rel = qlen - (taps - 1) + i;
      if (rel >= 0) val[i] = x[(int64_t)(t0 + rel) * ldx + c];
      else if (carried) val[i] = st[(int64_t)(taps - 1 + rel) * C + c];
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
    if (i < taps - 1) st[(int64_t)i * C + c] = val[i];
}

// ------------------------------------------------------------------------------------------------ recurrent state scan
enum ScanMode : int { SCAN_DECAY = 0, SCAN_DELTA = 1, SCAN_GATED = 2 };
enum GateKind : int { GATE_STEP = 1, GATE_EXP = 2, GATE_HEAD = 3 };
constexpr int SCAN_TOK_TILE = 8;

struct ScanParams {
  const void *q, *k, *v;        // [T, ld*]: q/k hold qk_heads x dim, v holds heads x vdim
  int64_t ldq, ldk, ldv;
  const void* araw;             // delta: pre-activation of the decay [T, lda] (heads x dim; heads with GATE_HEAD)
  int64_t lda;
  const void* braw;             // delta: pre-activation of the write strength [T, ldb] (heads)
  int64_t ldb;
  const float* head_decay;      // decay mode: [heads]
  const float* a_log;           // delta: [heads]
  const float* dt_bias;         // delta: [heads x dim]
  float* state;                 // [slots, heads, dim, vdim] fp32
  float* out;                   // [T, heads x vdim] fp32
  const int *cu_q, *ctx_len, *slots;
  int heads, qk_heads, dim, vdim;
  int act_silu;                 // silu on q, k, v when they are loaded
  int unit_qk;                  // q, k divided by sqrt(sum x^2 + unit_eps) per head
  float unit_eps, q_scale;
  float k_scale;                // k multiplied by this (after the rotation)
  const float* rot_table;       // [positions, rot_dims] cos | sin per position, or null: no rotary positions
  int rot_dims;                 // first channels of every q / k head that are rotated (pairs i, i + rot_dims / 2)
  const int* token_pos;         // [T] position of every token in its sequence
  // gated mode.  GATE_STEP (selective state space): araw [T, lda] holds heads step pre-activations, dt_bias / a_log
  // [heads]: step = softplus(araw + dt_bias), decay = exp(-exp(a_log) step), write strength = step; head_decay [heads]
  // (optional) is the skip D of y += D v.  GATE_EXP (matrix memory with exponential gates): araw holds heads input-gate
  // then heads forget-gate pre-activations, dt_bias [2 heads] their biases, gate_cap the soft cap (0 = none); the running
  // maximum and the normaliser vector live in state_m [slots, heads] / state_n [slots, heads, dim].
  int gate_kind;
  float gate_cap;
  float* state_n;
  float* state_m;
};

// Two kernels.  `scan_prepare_kernel` is elementwise and fully parallel: activations, unit norms, decays and write
// strengths of every token in fp32 into a workspace whose rows are padded to the kernel's key width (q, k: zeros;
// decay: ones) and value rows to a multiple of SCAN_COLS.  `state_scan_kernel` is the recurrence: a CTA owns SCAN_COLS
// value columns of one (sequence, head); column j of S lives in the registers of SCAN_PARTS adjacent lanes, each holding
// DK / SCAN_PARTS of its rows, so S^T k and S^T q are partial sums per lane joined by two shuffles in a fixed order.
// The workspace rows of SCAN_TOK_TILE tokens arrive by cp.async in a two-stage ring while the previous tile is walked.
constexpr int SCAN_PARTS = 4;
constexpr int SCAN_COLS = 32;          // 128 threads

struct ScanWork {
  float *q, *k, *g, *beta, *v;         // [T, qk_heads, DK] x2, [T, heads, DK], [T, heads], [T, heads, VP]
  float* gw;                           // gated mode: [T, heads, 4] = decay, write strength, read-out factor, unused
  int DK, VP;
};

CB_DEVICE void cp_async16f(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

template <int MODE, typename T>
__global__ void __launch_bounds__(128) scan_prepare_kernel(ScanParams p, ScanWork w) {
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dim = p.dim, vdim = p.vdim, DK = w.DK;
  const T* q = (const T*)p.q + t * p.ldq;
  const T* k = (const T*)p.k + t * p.ldk;
  for (int hk = warp; hk < p.qk_heads; hk += nwarps) {
    float* wq = w.q + (t * p.qk_heads + hk) * DK;
    float* wk = w.k + (t * p.qk_heads + hk) * DK;
    float ssq = 0.f, ssk = 0.f;
    for (int i = lane; i < dim; i += 32) {
      float qv = to_f32<T>(q[hk * dim + i]), kv = to_f32<T>(k[hk * dim + i]);
      if (p.act_silu) { qv = silu_f(qv); kv = silu_f(kv); }
      ssq = fmaf(qv, qv, ssq);
      ssk = fmaf(kv, kv, ssk);
      wq[i] = qv;
      wk[i] = kv;
    }
    if (p.rot_table != nullptr && p.rot_dims > 0) {      // a lane turns whole pairs: both halves are its own afterwards
      __syncwarp();
      const int half = p.rot_dims >> 1;
      const float* cs = p.rot_table + (int64_t)p.token_pos[t] * p.rot_dims;
      for (int i = lane; i < half; i += 32) {
        const float c = cs[i], sn = cs[half + i];
        const float qu = wq[i], qv = wq[i + half], ku = wk[i], kv = wk[i + half];
        wq[i] = qu * c - qv * sn;
        wq[i + half] = qv * c + qu * sn;
        wk[i] = ku * c - kv * sn;
        wk[i + half] = kv * c + ku * sn;
      }
      __syncwarp();
    }
    float rq = p.q_scale, rk = p.k_scale;
    if (p.unit_qk) {
      rq = p.q_scale / sqrtf(warp_sum(ssq) + p.unit_eps);
      rk = p.k_scale / sqrtf(warp_sum(ssk) + p.unit_eps);
    }
    for (int i = lane; i < DK; i += 32) {      // a lane rescales what it wrote itself; the padding is zero
      wq[i] = i < dim ? wq[i] * rq : 0.f;
      wk[i] = i < dim ? wk[i] * rk : 0.f;
    }
  }
  if (MODE == SCAN_DELTA) {
    for (int h = warp; h < p.heads; h += nwarps) {
      const float A = expf(p.a_log[h]);
      // GATE_HEAD: one decay per head (araw [T, heads], dt_bias [heads]) fills the head's row of channel decays
      const float gh = p.gate_kind == GATE_HEAD
                           ? expf(-A * softplus_f(to_f32<T>(((const T*)p.araw)[t * p.lda + h]) + p.dt_bias[h])) : 1.f;
      for (int i = lane; i < DK; i += 32) {
        float g = 1.f;
        if (i < dim)
          g = p.gate_kind == GATE_HEAD ? gh
              : expf(-A * softplus_f(to_f32<T>(((const T*)p.araw)[t * p.lda + h * dim + i]) + p.dt_bias[h * dim + i]));
        w.g[(t * p.heads + h) * DK + i] = g;
      }
    }
    for (int h = threadIdx.x; h < p.heads; h += blockDim.x)
      w.beta[t * p.heads + h] = sigmoid_f(to_f32<T>(((const T*)p.braw)[t * p.ldb + h]));
  }
  if (MODE == SCAN_GATED) {
    const T* ar = (const T*)p.araw + t * p.lda;
    for (int h = threadIdx.x; h < p.heads; h += blockDim.x) {
      float4 o;
      if (p.gate_kind == GATE_STEP) {
        const float step = softplus_f(to_f32<T>(ar[h]) + p.dt_bias[h]);
        o = make_float4(expf(-expf(p.a_log[h]) * step), step, 1.f, 0.f);
      } else {                                   // log forget gate, log input gate: the gate kernel turns them into
        float zi = to_f32<T>(ar[h]) + p.dt_bias[h];              // decay and write strength
        float zf = to_f32<T>(ar[p.heads + h]) + p.dt_bias[p.heads + h];
        if (p.gate_cap > 0.f) {
          zi = p.gate_cap * tanhf(zi / p.gate_cap);
          zf = p.gate_cap * tanhf(zf / p.gate_cap);
        }
        o = make_float4(logsigmoid_f(zf), zi, 1.f, 0.f);
      }
      *reinterpret_cast<float4*>(w.gw + (t * p.heads + h) * 4) = o;
    }
  }
  const T* v = (const T*)p.v + t * p.ldv;
  for (int idx = threadIdx.x; idx < p.heads * w.VP; idx += blockDim.x) {
    const int h = idx / w.VP, c = idx % w.VP;
    float vv = c < vdim ? to_f32<T>(v[h * vdim + c]) : 0.f;
    if (p.act_silu) vv = silu_f(vv);
    w.v[t * p.heads * w.VP + idx] = vv;
  }
}

// Matrix memory with exponential gates, the scalar side: one warp per (sequence, head) walks the portion's tokens with the
// running maximum m and the normaliser n (rows spread over the lanes): m' = max(f + m, i); decay = exp(f + m - m'),
// write = exp(i - m'); n <- decay n + write k; read-out factor = 1 / (max(|n . q|, exp(-m')) + 1e-6).  The three replace
// (f, i) in the workspace, where the matrix recurrence reads them.  Loads of the next token are issued before the
// current one's reduction.
template <int DK>
__global__ void __launch_bounds__(128) exp_gate_kernel(ScanParams p, ScanWork w, int nseq) {
  constexpr int NR = DK >= 32 ? DK / 32 : 1;
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= nseq * p.heads) return;
  const int s = unit / p.heads, h = unit % p.heads;
  const int t0 = p.cu_q[s], t1 = p.cu_q[s + 1];
  if (t0 >= t1) return;
  const bool carried = p.ctx_len[s] > 0;
  const int hk = h / (p.heads / p.qk_heads);
  float* ng = p.state_n + ((int64_t)p.slots[s] * p.heads + h) * p.dim;
  float* mg = p.state_m + (int64_t)p.slots[s] * p.heads + h;
  float n[NR], kc[NR], qc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int r = lane + 32 * i;
    n[i] = (carried && r < p.dim) ? ng[r] : 0.f;
    kc[i] = r < DK ? w.k[((int64_t)t0 * p.qk_heads + hk) * DK + r] : 0.f;
    qc[i] = r < DK ? w.q[((int64_t)t0 * p.qk_heads + hk) * DK + r] : 0.f;
  }
  float m = carried ? *mg : 0.f;
  float4 cur = *reinterpret_cast<const float4*>(w.gw + ((int64_t)t0 * p.heads + h) * 4);
  for (int64_t t = t0; t < t1; ++t) {
    float kn[NR], qn[NR];
    float4 nxt = cur;
    if (t + 1 < t1) {
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = lane + 32 * i;
        kn[i] = r < DK ? w.k[((t + 1) * p.qk_heads + hk) * DK + r] : 0.f;
        qn[i] = r < DK ? w.q[((t + 1) * p.qk_heads + hk) * DK + r] : 0.f;
      }
      nxt = *reinterpret_cast<const float4*>(w.gw + ((t + 1) * p.heads + h) * 4);
    }
    const float f = cur.x, ig = cur.y;
    const float mn = fmaxf(f + m, ig);
    const float dec = expf(f + m - mn), wr = expf(ig - mn);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      n[i] = fmaf(dec, n[i], wr * kc[i]);
      dot = fmaf(n[i], qc[i], dot);
    }
    dot = warp_sum(dot);
    m = mn;
    const float inv = 1.f / (fmaxf(fabsf(dot), expf(-m)) + 1e-6f);
    if (lane == 0) *reinterpret_cast<float4*>(w.gw + (t * p.heads + h) * 4) = make_float4(dec, wr, inv, 0.f);
    if (t + 1 < t1) {
#pragma unroll
      for (int i = 0; i < NR; ++i) { kc[i] = kn[i]; qc[i] = qn[i]; }
    }
    cur = nxt;
  }
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int r = lane + 32 * i;
    if (r < p.dim) ng[r] = n[i];
  }
  if (lane == 0) *mg = m;
}

template <int DK, int MODE>
__global__ void __launch_bounds__(128, DK > 128 ? 2 : 4) state_scan_kernel(ScanParams p, ScanWork w) {
  constexpr int RP = DK / SCAN_PARTS;  // rows per lane
  constexpr int RPP = RP + 4;          // a lane's rows start 4 floats further: the four 16-byte reads of a warp hit
  constexpr int DKP = SCAN_PARTS * RPP;  // different banks
  constexpr int NROW = MODE == SCAN_DELTA ? 3 : 2;
  constexpr int STAGE = SCAN_TOK_TILE * (NROW * DKP + SCAN_COLS + 4);     // floats per stage
  extern __shared__ __align__(16) float scan_smem[];
  const int vblocks = w.VP / SCAN_COLS;
  const int h = blockIdx.x / vblocks, vb = blockIdx.x % vblocks;
  const int s = blockIdx.y;
  const int t0 = p.cu_q[s], t1 = p.cu_q[s + 1];
  if (t0 >= t1) return;
  const int part = threadIdx.x % SCAN_PARTS;
  const int col = threadIdx.x / SCAN_PARTS;
  const int j = vb * SCAN_COLS + col;
  const bool active = j < p.vdim;
  const int hk = h / (p.heads / p.qk_heads);
  const int dim = p.dim, vdim = p.vdim;
  const int r0 = part * RP, r0p = part * RPP;
  float* Sg = p.state + ((int64_t)p.slots[s] * p.heads + h) * dim * vdim;
  float S[RP];
  const bool carried = p.ctx_len[s] > 0;
#pragma unroll
  for (int i = 0; i < RP; ++i) S[i] = (carried && active && r0 + i < dim) ? Sg[(int64_t)(r0 + i) * vdim + j] : 0.f;
  const float hd = MODE == SCAN_DECAY ? p.head_decay[h] : 0.f;
  const float skip = (MODE == SCAN_GATED && p.head_decay != nullptr) ? p.head_decay[h] : 0.f;

  auto load_tile = [&](int stage, int tb) {
    float* base = scan_smem + stage * STAGE;
    const int nt = min(SCAN_TOK_TILE, t1 - tb);
    constexpr int CH = DK / 4;
    for (int idx = threadIdx.x; idx < nt * CH; idx += blockDim.x) {
      const int tt = idx / CH, c = (idx % CH) * 4;
      const int dst = tt * DKP + c + 4 * (c / RP);
      const int64_t t = tb + tt;
      cp_async16f(base + dst, w.q + (t * p.qk_heads + hk) * DK + c);
      cp_async16f(base + SCAN_TOK_TILE * DKP + dst, w.k + (t * p.qk_heads + hk) * DK + c);
      if (MODE == SCAN_DELTA) cp_async16f(base + 2 * SCAN_TOK_TILE * DKP + dst, w.g + (t * p.heads + h) * DK + c);
    }
    float* sv = base + NROW * SCAN_TOK_TILE * DKP;
    for (int idx = threadIdx.x; idx < nt * (SCAN_COLS / 4); idx += blockDim.x) {
      const int tt = idx / (SCAN_COLS / 4), c = (idx % (SCAN_COLS / 4)) * 4;
      cp_async16f(sv + tt * SCAN_COLS + c, w.v + ((int64_t)(tb + tt) * p.heads + h) * w.VP + vb * SCAN_COLS + c);
    }
    if (MODE == SCAN_DELTA && threadIdx.x < nt)
      sv[SCAN_TOK_TILE * SCAN_COLS + threadIdx.x] = w.beta[(int64_t)(tb + threadIdx.x) * p.heads + h];
    if (MODE == SCAN_GATED && threadIdx.x < nt)
      cp_async16f(sv + SCAN_TOK_TILE * SCAN_COLS + threadIdx.x * 4,
                  w.gw + ((int64_t)(tb + threadIdx.x) * p.heads + h) * 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  load_tile(0, t0);
  int stage = 0;
  for (int tb = t0; tb < t1; tb += SCAN_TOK_TILE, stage ^= 1) {
    const int nt = min(SCAN_TOK_TILE, t1 - tb);
    if (tb + SCAN_TOK_TILE < t1) {              // the other stage was released by the barrier that ended the last pass
      load_tile(stage ^ 1, tb + SCAN_TOK_TILE);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* sq = scan_smem + stage * STAGE;
    const float* sk = sq + SCAN_TOK_TILE * DKP;
    const float* sg = sk + SCAN_TOK_TILE * DKP;
    const float* sv = sq + NROW * SCAN_TOK_TILE * DKP;
    const float* sbeta = sv + SCAN_TOK_TILE * SCAN_COLS;
    for (int tt = 0; tt < nt; ++tt) {            // every lane takes part in the shuffles, also for a padded column
      const int64_t t = tb + tt;
      const float vv = sv[tt * SCAN_COLS + col];
      const float* kq = sk + tt * DKP + r0p;
      const float* qq = sq + tt * DKP + r0p;
      float o0 = 0.f, o1 = 0.f;
      float4 gwv = make_float4(0.f, 0.f, 1.f, 0.f);
      if (MODE == SCAN_GATED) {
        gwv = *reinterpret_cast<const float4*>(sbeta + tt * 4);
        const float u = gwv.y * vv;
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
          S[i] = fmaf(gwv.x, S[i], k4.x * u); S[i + 1] = fmaf(gwv.x, S[i + 1], k4.y * u);
          S[i + 2] = fmaf(gwv.x, S[i + 2], k4.z * u); S[i + 3] = fmaf(gwv.x, S[i + 3], k4.w * u);
          o0 = fmaf(S[i], q4.x, o0); o1 = fmaf(S[i + 1], q4.y, o1);
          o0 = fmaf(S[i + 2], q4.z, o0); o1 = fmaf(S[i + 3], q4.w, o1);
        }
      } else if (MODE == SCAN_DELTA) {
        const float* gq = sg + tt * DKP + r0p;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(gq + i);
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
          a0 = fmaf(S[i], k4.x, a0); a1 = fmaf(S[i + 1], k4.y, a1);
          a0 = fmaf(S[i + 2], k4.z, a0); a1 = fmaf(S[i + 3], k4.w, a1);
        }
        float kv = a0 + a1;
        kv += __shfl_xor_sync(0xffffffffu, kv, 1);
        kv += __shfl_xor_sync(0xffffffffu, kv, 2);
        const float u = sbeta[tt] * (vv - kv);
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
          S[i] = fmaf(k4.x, u, S[i]); S[i + 1] = fmaf(k4.y, u, S[i + 1]);
          S[i + 2] = fmaf(k4.z, u, S[i + 2]); S[i + 3] = fmaf(k4.w, u, S[i + 3]);
          o0 = fmaf(S[i], q4.x, o0); o1 = fmaf(S[i + 1], q4.y, o1);
          o0 = fmaf(S[i + 2], q4.z, o0); o1 = fmaf(S[i + 3], q4.w, o1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < RP; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kq + i);
          const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
          S[i] = fmaf(hd, S[i], k4.x * vv); S[i + 1] = fmaf(hd, S[i + 1], k4.y * vv);
          S[i + 2] = fmaf(hd, S[i + 2], k4.z * vv); S[i + 3] = fmaf(hd, S[i + 3], k4.w * vv);
          o0 = fmaf(S[i], q4.x, o0); o1 = fmaf(S[i + 1], q4.y, o1);
          o0 = fmaf(S[i + 2], q4.z, o0); o1 = fmaf(S[i + 3], q4.w, o1);
        }
      }
      float o = o0 + o1;
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (MODE == SCAN_GATED) o = fmaf(o, gwv.z, skip * vv);
      if (active && part == 0) p.out[t * ((int64_t)p.heads * vdim) + h * vdim + j] = o;
    }
    __syncthreads();                            // this stage may be refilled in the next pass
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < RP; ++i)
      if (r0 + i < dim) Sg[(int64_t)(r0 + i) * vdim + j] = S[i];
  }
}

template <int DK, int MODE> int launch_scan_dk(const ScanParams& p, const ScanWork& w, int nseq, cudaStream_t st) {
  constexpr int DKP = SCAN_PARTS * (DK / SCAN_PARTS + 4);
  constexpr int NROW = MODE == SCAN_DELTA ? 3 : 2;
  const size_t smem = (size_t)2 * SCAN_TOK_TILE * (NROW * DKP + SCAN_COLS + 4) * sizeof(float);
  auto kern = state_scan_kernel<DK, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  dim3 grid(p.heads * (w.VP / SCAN_COLS), nseq);
  kern<<<grid, SCAN_COLS * SCAN_PARTS, smem, st>>>(p, w);
  return CB_LAUNCH_CHECK();
}

// workspace floats for `tokens` tokens: q, k rows, decay rows and write strengths (delta rule), value rows
static inline int scan_dk(int dim) { return dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256; }
static inline int scan_vp(int vdim) { return (vdim + SCAN_COLS - 1) / SCAN_COLS * SCAN_COLS; }

template <int MODE, typename T>
int launch_scan(const ScanParams& p, float* work, int64_t tokens, int nseq, cudaStream_t st) {
  if (p.dim > 256) return (int)cudaErrorInvalidValue;
  ScanWork w;
  w.DK = scan_dk(p.dim);
  w.VP = scan_vp(p.vdim);
  w.q = work;
  w.k = w.q + tokens * p.qk_heads * w.DK;
  w.g = w.k + tokens * p.qk_heads * w.DK;
  w.beta = w.g + (MODE == SCAN_DELTA ? tokens * p.heads * w.DK : 0);
  w.gw = w.beta;
  w.v = w.beta + (MODE == SCAN_DELTA ? (tokens * p.heads + 3) / 4 * 4 : (MODE == SCAN_GATED ? tokens * p.heads * 4 : 0));
  scan_prepare_kernel<MODE, T><<<(unsigned)tokens, 128, 0, st>>>(p, w);
  if (MODE == SCAN_GATED && p.gate_kind == GATE_EXP) {
    const unsigned blocks = (unsigned)((nseq * p.heads + 3) / 4);
    if (w.DK == 16) exp_gate_kernel<16><<<blocks, 128, 0, st>>>(p, w, nseq);
    else if (w.DK == 32) exp_gate_kernel<32><<<blocks, 128, 0, st>>>(p, w, nseq);
    else if (w.DK == 64) exp_gate_kernel<64><<<blocks, 128, 0, st>>>(p, w, nseq);
    else if (w.DK == 128) exp_gate_kernel<128><<<blocks, 128, 0, st>>>(p, w, nseq);
    else exp_gate_kernel<256><<<blocks, 128, 0, st>>>(p, w, nseq);
  }
  if (w.DK == 16) return launch_scan_dk<16, MODE>(p, w, nseq, st);
  if (w.DK == 32) return launch_scan_dk<32, MODE>(p, w, nseq, st);
  if (w.DK == 64) return launch_scan_dk<64, MODE>(p, w, nseq, st);
  if (w.DK == 128) return launch_scan_dk<128, MODE>(p, w, nseq, st);
  return launch_scan_dk<256, MODE>(p, w, nseq, st);
}

// ------------------------------------------------------------------------------------------------ norms
// one warp per (token, group): out = o / sqrt(mean_group(o^2) + eps) * w[c % wn] * act(gate), act = sigmoid or silu;
// w and gate are optional
template <typename T>
__global__ void __launch_bounds__(256) gated_group_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ w,
                                                                  int wn, const T* __restrict__ gate, int64_t ldg,
                                                                  T* __restrict__ out, int64_t tokens, int C, int group,
                                                                  float eps, int flags) {
  const bool gate_silu = flags & 1;
  const bool gate_first = (flags & 2) && gate != nullptr;      // the gate multiplies o before the norm
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int ngroups = C / group;
  if (unit >= tokens * ngroups) return;
  const int64_t t = unit / ngroups;
  const int c0 = (int)(unit % ngroups) * group;
  const float* row = o + t * C + c0;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) {
    float v = row[i];
    if (gate_first) {
      const float gv = to_f32<T>(gate[t * ldg + c0 + i]);
      v *= gate_silu ? silu_f(gv) : sigmoid_f(gv);
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32) {
    const int c = c0 + i;
    float y = row[i];
    if (gate_first) {
      const float gv = to_f32<T>(gate[t * ldg + c]);
      y *= gate_silu ? silu_f(gv) : sigmoid_f(gv);
    }
    y *= r;
    if (w != nullptr) y *= to_f32<T>(w[c % wn]);
    if (gate != nullptr && !gate_first) {
      const float gv = to_f32<T>(gate[t * ldg + c]);
      y *= gate_silu ? silu_f(gv) : sigmoid_f(gv);
    }
    out[t * C + c] = from_f32<T>(y);
  }
}

// wide groups (a state space's whole inner width is one group): one CTA per (token, group), four channels per thread and
// step (16-byte reads of o, 8-byte ones of 16-bit operands; the launcher checks widths and alignment)
template <typename T>
__global__ void __launch_bounds__(256) gated_group_rmsnorm_wide_kernel(const float* __restrict__ o, const T* __restrict__ w,
                                                                       int wn, const T* __restrict__ gate, int64_t ldg,
                                                                       T* __restrict__ out, int C, int group, float eps,
                                                                       int flags) {
  struct alignas(sizeof(T) * 4) Pack { T v[4]; };
  __shared__ float red[32];
  const bool gate_silu = flags & 1;
  const bool gate_first = (flags & 2) && gate != nullptr;
  const int ngroups = C / group;
  const int64_t t = blockIdx.x / ngroups;
  const int c0 = (int)(blockIdx.x % ngroups) * group;
  const float* row = o + t * C + c0;
  const T* grow = gate != nullptr ? gate + t * ldg + c0 : nullptr;
  float ss[1] = {0.f};
  for (int i = threadIdx.x * 4; i < group; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(row + i);
    if (gate_first) {
      const Pack g = *reinterpret_cast<const Pack*>(grow + i);
      const float g0 = to_f32<T>(g.v[0]), g1 = to_f32<T>(g.v[1]), g2 = to_f32<T>(g.v[2]), g3 = to_f32<T>(g.v[3]);
      v.x *= gate_silu ? silu_f(g0) : sigmoid_f(g0); v.y *= gate_silu ? silu_f(g1) : sigmoid_f(g1);
      v.z *= gate_silu ? silu_f(g2) : sigmoid_f(g2); v.w *= gate_silu ? silu_f(g3) : sigmoid_f(g3);
    }
    ss[0] = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss[0]))));
  }
  block_sum<1>(ss, red);
  const float r = 1.f / sqrtf(ss[0] / (float)group + eps);
  for (int i = threadIdx.x * 4; i < group; i += blockDim.x * 4) {
    const float4 v4 = *reinterpret_cast<const float4*>(row + i);
    float v[4] = {v4.x, v4.y, v4.z, v4.w};
    Pack g, res;
    if (gate != nullptr) g = *reinterpret_cast<const Pack*>(grow + i);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float y = v[e];
      const float gv = gate != nullptr ? to_f32<T>(g.v[e]) : 0.f;
      const float ga = gate_silu ? silu_f(gv) : sigmoid_f(gv);
      if (gate_first) y *= ga;
      y *= r;
      if (w != nullptr) y *= to_f32<T>(w[(c0 + i + e) % wn]);
      if (gate != nullptr && !gate_first) y *= ga;
      res.v[e] = from_f32<T>(y);
    }
    *reinterpret_cast<Pack*>(out + t * C + c0 + i) = res;
  }
}

// one CTA per (token row, norm group).  x (fp32) += mult * y / rms_group(y) * (offset + w); h = cast(x): the row is cut into
// `groups` equal consecutive parts and every part is divided by its own root mean square.  y is the 16-bit type T or
// (TY = float) an fp32 sum.  VEC = 4: 16-byte accesses of the stream, 8-byte ones of 16-bit operands (group width and
// strides multiples of 4, checked by the launcher).
//
// With `hist` the updated x is slice n - 1 of a stream history [n, T x W] (slices `hstride` apart) and the kernel goes on
// to the weighted sum over the history, mix = sum_j coef[j] hist[j] (j ascending, the new x last), written to `mix_out`
// in fp32; h is then cast(mix) instead of cast(x): the layer's last sublayer and the depth average in one pass.
template <typename T, typename TY, int VEC>
__global__ void __launch_bounds__(256) rmsnorm_residual_kernel(float* __restrict__ x, const TY* __restrict__ y, int64_t ldy,
                                                               const T* __restrict__ w, T* __restrict__ h, int W,
                                                               int groups, float eps, float mult, float offset,
                                                               const float* __restrict__ hist, int64_t hstride, int n,
                                                               const float* __restrict__ coef,
                                                               float* __restrict__ mix_out) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  struct alignas(sizeof(TY) * VEC) PackY { TY v[VEC]; };
  struct alignas(sizeof(float) * VEC) PackF { float v[VEC]; };
  __shared__ float red[64];
  const int64_t t = blockIdx.x / groups;
  const int Wg = W / groups, c0 = (int)(blockIdx.x % groups) * Wg;
  const TY* yr = y + t * ldy + c0;
  float ss[1] = {0.f};
  // a group that the CTA covers in one step (the usual case): the stream's and the weight's loads are issued together
  // with y's, ahead of the reduction, so that one round trip to memory serves the whole row
  const bool one_step = Wg <= (int)blockDim.x * VEC;
  const int i0 = threadIdx.x * VEC;
  PackY a0;
  Pack w0;
  PackF x0;
  if (one_step && i0 < Wg) {
    a0 = *reinterpret_cast<const PackY*>(yr + i0);
    w0 = *reinterpret_cast<const Pack*>(w + c0 + i0);
    x0 = *reinterpret_cast<const PackF*>(x + t * W + c0 + i0);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ss[0] = fmaf(to_f32<TY>(a0.v[e]), to_f32<TY>(a0.v[e]), ss[0]);
  }
  if (!one_step) {
    for (int i = threadIdx.x * VEC; i < Wg; i += blockDim.x * VEC) {
      const PackY a = *reinterpret_cast<const PackY*>(yr + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss[0] = fmaf(to_f32<TY>(a.v[e]), to_f32<TY>(a.v[e]), ss[0]);
    }
  }
  block_sum<1>(ss, red);
  const float r = 1.f / sqrtf(ss[0] / (float)Wg + eps);
  for (int i = threadIdx.x * VEC; i < Wg; i += blockDim.x * VEC) {
    const PackY a = one_step ? a0 : *reinterpret_cast<const PackY*>(yr + i);
    const Pack ww = one_step ? w0 : *reinterpret_cast<const Pack*>(w + c0 + i);
    PackF xv = one_step ? x0 : *reinterpret_cast<const PackF*>(x + t * W + c0 + i);
    Pack hv;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      xv.v[e] += mult * (to_f32<TY>(a.v[e]) * r * (offset + to_f32<T>(ww.v[e])));
      hv.v[e] = from_f32<T>(xv.v[e]);
    }
    *reinterpret_cast<PackF*>(x + t * W + c0 + i) = xv;
    if (hist != nullptr) {
      PackF acc;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] = 0.f;
      for (int j = 0; j + 1 < n; ++j) {
        const float cj = __ldg(coef + j);
        const PackF hj = *reinterpret_cast<const PackF*>(hist + j * hstride + t * W + c0 + i);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc.v[e] = fmaf(cj, hj.v[e], acc.v[e]);
      }
      const float cl = __ldg(coef + n - 1);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        acc.v[e] = fmaf(cl, xv.v[e], acc.v[e]);
        hv.v[e] = from_f32<T>(acc.v[e]);
      }
      *reinterpret_cast<PackF*>(mix_out + t * W + c0 + i) = acc;
    }
    if (h != nullptr) *reinterpret_cast<Pack*>(h + t * W + c0 + i) = hv;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_f32in_kernel(const float* __restrict__ x, int64_t ldx,
                                                            const T* __restrict__ w, T* __restrict__ out, int W,
                                                            int groups, float eps, float offset) {
  __shared__ float red[64];
  const int64_t t = blockIdx.x / groups;
  const int Wg = W / groups, c0 = (int)(blockIdx.x % groups) * Wg;
  const float* xr = x + t * ldx + c0;
  float ss[1] = {0.f};
  for (int i = threadIdx.x; i < Wg; i += blockDim.x) ss[0] = fmaf(xr[i], xr[i], ss[0]);
  block_sum<1>(ss, red);
  const float r = 1.f / sqrtf(ss[0] / (float)Wg + eps);
  for (int i = threadIdx.x; i < Wg; i += blockDim.x)
    out[t * W + c0 + i] = from_f32<T>(xr[i] * r * (offset + to_f32<T>(w[c0 + i])));
}

// Weighted sum over the history of an fp32 residual stream: hist [n, T x W] (slices `stride` elements apart),
// out = sum_j coef[j] hist[j] in ascending j (coef: n fp32 numbers on the device), written as fp32 and (optionally) in
// the compute dtype for the next layer's GEMMs.  Four elements per thread, all n loads of a thread independent.
template <typename T>
__global__ void __launch_bounds__(256) depth_mix_kernel(const float* __restrict__ hist, int64_t stride, int n,
                                                        const float* __restrict__ coef, float* __restrict__ out,
                                                        T* __restrict__ h, int64_t total4) {
  struct alignas(sizeof(T) * 4) Pack { T v[4]; };
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n; ++j) {
      const float a = __ldg(coef + j);
      const float4 v = *reinterpret_cast<const float4*>(hist + j * stride + i * 4);
      acc.x = fmaf(a, v.x, acc.x); acc.y = fmaf(a, v.y, acc.y); acc.z = fmaf(a, v.z, acc.z); acc.w = fmaf(a, v.w, acc.w);
    }
    *reinterpret_cast<float4*>(out + i * 4) = acc;
    if (h != nullptr) {
      Pack p;
      p.v[0] = from_f32<T>(acc.x); p.v[1] = from_f32<T>(acc.y); p.v[2] = from_f32<T>(acc.z); p.v[3] = from_f32<T>(acc.w);
      *reinterpret_cast<Pack*>(h + i * 4) = p;
    }
  }
}

// Polynomial activation with normalised powers, one CTA per token row: out = a N(z) + b N(z^2) + c N(z^3) + e with powers
// taken element by element and N(u) = u / sqrt(mean(u^2) + eps) over the row; the three sums of squares (z^2, z^4, z^6)
// come from one pass, everything in fp32.  coef = (a, b, c, e) on the device.  VEC elements per access (16 bytes when the
// row allows); the first POLY_ITEMS vectors of a thread stay in registers between the two passes, so rows up to
// threads x POLY_ITEMS x VEC wide (16384 16-bit values with 512 threads) are read once - all their loads in flight
// together - and wider ones re-read the rest.
template <typename T, int VEC, int POLY_ITEMS>
__global__ void __launch_bounds__(512) poly_norm_kernel(const T* __restrict__ z, int64_t ldz, T* __restrict__ out, int F,
                                                        const float* __restrict__ coef, float eps) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  __shared__ float red[3 * 32];
  const int64_t t = blockIdx.x;
  const T* zr = z + t * ldz;
  const int step = blockDim.x * VEC;
  Pack keep[POLY_ITEMS];
#pragma unroll
  for (int it = 0; it < POLY_ITEMS; ++it) {
    const int i = threadIdx.x * VEC + it * step;
    if (i < F) keep[it] = *reinterpret_cast<const Pack*>(zr + i);
  }
  float ss[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int it = 0; it < POLY_ITEMS; ++it) {
    if (threadIdx.x * VEC + it * step < F) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float v = to_f32<T>(keep[it].v[e]), v2 = v * v;
        ss[0] += v2;
        ss[1] = fmaf(v2, v2, ss[1]);
        ss[2] = fmaf(v2 * v, v2 * v, ss[2]);
      }
    }
  }
  for (int i = threadIdx.x * VEC + POLY_ITEMS * step; i < F; i += step) {
    const Pack a = *reinterpret_cast<const Pack*>(zr + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float v = to_f32<T>(a.v[e]), v2 = v * v;
      ss[0] += v2;
      ss[1] = fmaf(v2, v2, ss[1]);
      ss[2] = fmaf(v2 * v, v2 * v, ss[2]);
    }
  }
  block_sum<3>(ss, red);
  const float r1 = coef[0] / sqrtf(ss[0] / (float)F + eps), r2 = coef[1] / sqrtf(ss[1] / (float)F + eps),
              r3 = coef[2] / sqrtf(ss[2] / (float)F + eps), e0 = coef[3];
#pragma unroll
  for (int it = 0; it < POLY_ITEMS; ++it) {
    const int i = threadIdx.x * VEC + it * step;
    if (i < F) {
      Pack o;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float v = to_f32<T>(keep[it].v[e]), v2 = v * v;
        o.v[e] = from_f32<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e0))));
      }
      *reinterpret_cast<Pack*>(out + t * F + i) = o;
    }
  }
  for (int i = threadIdx.x * VEC + POLY_ITEMS * step; i < F; i += step) {
    const Pack a = *reinterpret_cast<const Pack*>(zr + i);
    Pack o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float v = to_f32<T>(a.v[e]), v2 = v * v;
      o.v[e] = from_f32<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e0))));
    }
    *reinterpret_cast<Pack*>(out + t * F + i) = o;
  }
}

// RMS norm of every head of a [T, heads x dim] projection with one weight over the head's channels, shared by the heads:
// the first `heads_a` heads take `wa`, the others `wb` (query heads, then key heads).  One warp per (token, head), fp32;
// VEC channels per access, the first HEAD_ITEMS vectors of a lane stay in registers between the two passes (1: heads up
// to 32 x VEC channels, one load per lane and few registers; 8: wide rows such as a query latent).
// With `k_cache` the key heads do not go to `out`: the normed head is written into the token's row of the paged key cache
// [blocks, block_size, heads_b, dim] and the head as it came in (before the norm) into the same place of `v_cache` -
// attention whose values are its un-normed keys gets its query tile and both pages from one pass.
template <typename T, int VEC, int HEAD_ITEMS>
__global__ void __launch_bounds__(128) head_rmsnorm_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ out,
                                                           int64_t ldo, int64_t tokens, int heads, int heads_a, int dim,
                                                           const T* __restrict__ wa, const T* __restrict__ wb, float eps,
                                                           T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                           const int* __restrict__ block_tables,
                                                           const int* __restrict__ token_seq,
                                                           const int* __restrict__ token_pos, int block_size,
                                                           int max_blocks) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= tokens * heads) return;
  const int64_t t = unit / heads;
  const int hd = (int)(unit % heads);
  const T* row = x + t * ldx + hd * dim;
  const T* w = hd < heads_a ? wa : wb;
  Pack keep[HEAD_ITEMS];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < HEAD_ITEMS; ++it) {
    const int i = (lane + 32 * it) * VEC;
    if (i < dim) {
      keep[it] = *reinterpret_cast<const Pack*>(row + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) { const float v = to_f32<T>(keep[it].v[e]); ss = fmaf(v, v, ss); }
    }
  }
  for (int i = (lane + 32 * HEAD_ITEMS) * VEC; i < dim; i += 32 * VEC) {
    const Pack a = *reinterpret_cast<const Pack*>(row + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) { const float v = to_f32<T>(a.v[e]); ss = fmaf(v, v, ss); }
  }
  const float r = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
  T* orow = out + t * ldo + hd * dim;
  T* vrow = nullptr;
  if (k_cache != nullptr && hd >= heads_a) {
    const int seq = token_seq[t], pos = token_pos[t];
    const int64_t prow = (int64_t)block_tables[(int64_t)seq * max_blocks + pos / block_size] * block_size + pos % block_size;
    const int64_t at = (prow * (heads - heads_a) + (hd - heads_a)) * dim;
    orow = k_cache + at;
    vrow = v_cache + at;
  }
#pragma unroll
  for (int it = 0; it < HEAD_ITEMS; ++it) {
    const int i = (lane + 32 * it) * VEC;
    if (i < dim) {
      const Pack ww = *reinterpret_cast<const Pack*>(w + i);
      Pack o;
#pragma unroll
      for (int e = 0; e < VEC; ++e) o.v[e] = from_f32<T>(to_f32<T>(keep[it].v[e]) * r * to_f32<T>(ww.v[e]));
      *reinterpret_cast<Pack*>(orow + i) = o;
      if (vrow != nullptr) *reinterpret_cast<Pack*>(vrow + i) = keep[it];
    }
  }
  for (int i = (lane + 32 * HEAD_ITEMS) * VEC; i < dim; i += 32 * VEC) {
    const Pack a = *reinterpret_cast<const Pack*>(row + i);
    const Pack ww = *reinterpret_cast<const Pack*>(w + i);
    Pack o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) o.v[e] = from_f32<T>(to_f32<T>(a.v[e]) * r * to_f32<T>(ww.v[e]));
    *reinterpret_cast<Pack*>(orow + i) = o;
    if (vrow != nullptr) *reinterpret_cast<Pack*>(vrow + i) = a;
  }
}

// ------------------------------------------------------------------------------------------------ stream sums + norm
// One CTA per token row of the fp32 residual stream: x += ((a0 + a1) + a2 + a3) + row, every addend either fp32 or the
// 16-bit type T, summed among themselves first; then, with NORM = 1 / 2, h = cast(norm(x) * (offset + w)) where the norm
// is x / sqrt(mean x^2 + eps) or (x - mean) / sqrt(mean (x - mean)^2 + eps) (w and h: fp32 or T).  The row stays in
// registers between the passes: ITEMS x VEC values per thread, chosen by the launcher from the row width (rows wider
// than 8 x VEC x threads re-read the rest from x, which the same thread wrote).  Every load of the row is issued before
// the first store.
constexpr int STREAM_THREADS = 256;

struct StreamArgs {
  float* x;
  const void* a[4];
  int64_t ld[4];
  int a_f32[4];                 // addend j is fp32 (else T)
  const float* row;
  const void* w;
  int w_f32;
  void* h;
  int h_f32;
  int W;
  float eps, offset;
};

template <typename T, int VEC> CB_DEVICE void load_vec(const void* p, bool f32, int64_t i, float (&v)[VEC]) {
  if (f32) {
    struct alignas(4 * VEC) P { float e[VEC]; };
    const P a = *reinterpret_cast<const P*>((const float*)p + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = a.e[e];
  } else {
    struct alignas(sizeof(T) * VEC) P { T e[VEC]; };
    const P a = *reinterpret_cast<const P*>((const T*)p + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = to_f32<T>(a.e[e]);
  }
}
template <typename T, int VEC> CB_DEVICE void store_vec(void* p, bool f32, int64_t i, const float (&v)[VEC]) {
  if (f32) {
    struct alignas(4 * VEC) P { float e[VEC]; };
    P a;
#pragma unroll
    for (int e = 0; e < VEC; ++e) a.e[e] = v[e];
    *reinterpret_cast<P*>((float*)p + i) = a;
  } else {
    struct alignas(sizeof(T) * VEC) P { T e[VEC]; };
    P a;
#pragma unroll
    for (int e = 0; e < VEC; ++e) a.e[e] = from_f32<T>(v[e]);
    *reinterpret_cast<P*>((T*)p + i) = a;
  }
}

// new stream values of VEC columns starting at i: x + (sum of the addends + row)
template <typename T, int VEC> CB_DEVICE void stream_take(const StreamArgs& g, const float* xr, int64_t t, int i,
                                                          float (&xv)[VEC]) {
  float add[VEC];
  bool any = false;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (g.a[j] != nullptr) {
      float v[VEC];
      load_vec<T, VEC>(g.a[j], g.a_f32[j] != 0, t * g.ld[j] + i, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) add[e] = any ? add[e] + v[e] : v[e];
      any = true;
    }
  if (g.row != nullptr) {
    float v[VEC];
    load_vec<T, VEC>(g.row, true, i, v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) add[e] = any ? add[e] + v[e] : v[e];
    any = true;
  }
  load_vec<T, VEC>(xr, true, i, xv);
  if (any) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) xv[e] += add[e];
  }
}

template <typename T, int VEC, int ITEMS, int NORM>
__global__ void __launch_bounds__(STREAM_THREADS, ITEMS <= 2 ? 6 : (ITEMS <= 4 ? 4 : 3)) stream_add_norm_kernel(StreamArgs g) {
  constexpr int STEP = STREAM_THREADS * VEC;
  __shared__ float red[64];
  const int64_t t = blockIdx.x;
  const int W = g.W;
  float* xr = g.x + t * W;
  const bool any = g.a[0] != nullptr || g.a[1] != nullptr || g.a[2] != nullptr || g.a[3] != nullptr || g.row != nullptr;
  float keep[ITEMS][VEC];
  float sum[1] = {0.f};
  const int i0 = threadIdx.x * VEC;
#pragma unroll
  for (int n = 0; n < ITEMS; ++n) {
    const int i = i0 + n * STEP;
    if (i < W) {
      stream_take<T, VEC>(g, xr, t, i, keep[n]);
#pragma unroll
      for (int e = 0; e < VEC; ++e) sum[0] += NORM == 1 ? keep[n][e] * keep[n][e] : keep[n][e];
    }
  }
  if (any) {
#pragma unroll
    for (int n = 0; n < ITEMS; ++n)
      if (i0 + n * STEP < W) store_vec<T, VEC>(xr, true, i0 + n * STEP, keep[n]);
  }
  for (int i = i0 + ITEMS * STEP; i < W; i += STEP) {       // rows wider than the registers hold
    float xv[VEC];
    stream_take<T, VEC>(g, xr, t, i, xv);
    if (any) store_vec<T, VEC>(xr, true, i, xv);
#pragma unroll
    for (int e = 0; e < VEC; ++e) sum[0] += NORM == 1 ? xv[e] * xv[e] : xv[e];
  }
  if (NORM == 0) return;
  block_sum<1>(sum, red);
  float mean = 0.f, r;
  if (NORM == 1) {
    r = 1.f / sqrtf(sum[0] / (float)W + g.eps);
  } else {
    mean = sum[0] / (float)W;
    float sq[1] = {0.f};
#pragma unroll
    for (int n = 0; n < ITEMS; ++n)
      if (i0 + n * STEP < W) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { const float d = keep[n][e] - mean; sq[0] = fmaf(d, d, sq[0]); }
      }
    for (int i = i0 + ITEMS * STEP; i < W; i += STEP) {
      float xv[VEC];
      load_vec<T, VEC>(xr, true, i, xv);
#pragma unroll
      for (int e = 0; e < VEC; ++e) { const float d = xv[e] - mean; sq[0] = fmaf(d, d, sq[0]); }
    }
    block_sum<1>(sq, red);
    r = 1.f / sqrtf(sq[0] / (float)W + g.eps);
  }
  auto emit = [&](int i, const float (&xv)[VEC]) {
    float wv[VEC], y[VEC];
    if (g.w != nullptr) load_vec<T, VEC>(g.w, g.w_f32 != 0, i, wv);
#pragma unroll
    for (int e = 0; e < VEC; ++e) y[e] = (xv[e] - mean) * r * (g.offset + (g.w != nullptr ? wv[e] : 1.f));
    store_vec<T, VEC>(g.h, g.h_f32 != 0, t * W + i, y);
  };
#pragma unroll
  for (int n = 0; n < ITEMS; ++n)
    if (i0 + n * STEP < W) emit(i0 + n * STEP, keep[n]);
  for (int i = i0 + ITEMS * STEP; i < W; i += STEP) {
    float xv[VEC];
    load_vec<T, VEC>(xr, true, i, xv);
    emit(i, xv);
  }
}

template <typename T, int NORM> int launch_stream_add_norm(const StreamArgs& g, int64_t tokens, bool vec, cudaStream_t st) {
  const unsigned grid = (unsigned)tokens;
  if (!vec) stream_add_norm_kernel<T, 1, 8, NORM><<<grid, STREAM_THREADS, 0, st>>>(g);
  else if (g.W <= 2 * 4 * STREAM_THREADS) stream_add_norm_kernel<T, 4, 2, NORM><<<grid, STREAM_THREADS, 0, st>>>(g);
  else if (g.W <= 4 * 4 * STREAM_THREADS) stream_add_norm_kernel<T, 4, 4, NORM><<<grid, STREAM_THREADS, 0, st>>>(g);
  else stream_add_norm_kernel<T, 4, 8, NORM><<<grid, STREAM_THREADS, 0, st>>>(g);
  return CB_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------ rotary positions
// table [positions, dims] fp32: cos(p f_i) for i < dims / 2, then sin(p f_i).  A work item is VEC consecutive channels of
// one (token, head): in the rotated part the item takes channels i.. of the first half TOGETHER with their partners
// i + dims / 2.. (two loads, two stores of VEC values); behind the rotated part it copies.  VEC = 8 (16-byte accesses of
// 16-bit data) when every offset, stride and width allows it, else 1.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) rotary_half_kernel(const T* __restrict__ src, int64_t lds, T* __restrict__ dst,
                                                          int64_t ldd, int64_t tokens, int heads, int src_hs, int src_off,
                                                          int dst_hs, int dst_off, int width, int dims,
                                                          const float* __restrict__ table,
                                                          const int* __restrict__ token_pos) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  const int half = dims >> 1;
  const int items = (half + (width - dims)) / VEC;          // per (token, head): pair groups, then copy groups
  const int64_t total = tokens * heads * items;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int it = (int)(idx % items);
    const int h = (int)((idx / items) % heads);
    const int64_t t = idx / ((int64_t)items * heads);
    const T* s = src + t * lds + h * src_hs + src_off;
    T* d = dst + t * ldd + h * dst_hs + dst_off;
    const int c = it * VEC;
    if (c < half) {
      const float* cs = table + (int64_t)token_pos[t] * dims;
      const Pack u = *reinterpret_cast<const Pack*>(s + c);
      const Pack v = *reinterpret_cast<const Pack*>(s + c + half);
      Pack ou, ov;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float co = cs[c + e], sn = cs[half + c + e];
        const float uf = to_f32<T>(u.v[e]), vf = to_f32<T>(v.v[e]);
        ou.v[e] = from_f32<T>(uf * co - vf * sn);
        ov.v[e] = from_f32<T>(vf * co + uf * sn);
      }
      *reinterpret_cast<Pack*>(d + c) = ou;
      *reinterpret_cast<Pack*>(d + c + half) = ov;
    } else {
      const int cc = c + half;                               // the channel behind the rotated part
      *reinterpret_cast<Pack*>(d + cc) = *reinterpret_cast<const Pack*>(s + cc);
    }
  }
}

// One warp per token: the first `rank` columns of z are RMS-normalised with weight w (the latent), the last `rot` are
// turned by the token's position; both go into the token's row of the paged cache [blocks, block_size, 1, rank + rot].
// VEC = 8: a lane holds 8 adjacent latent columns per step in registers between the sum of squares and the store (16-byte
// accesses; the launcher checks widths and alignment), else VEC = 1.
template <typename T, typename TW, int VEC>
__global__ void __launch_bounds__(256) latent_kv_write_kernel(const T* __restrict__ z, int64_t ldz, const TW* __restrict__ w,
                                                              float eps, int rank, int rot,
                                                              const float* __restrict__ table, T* __restrict__ cache,
                                                              const int* __restrict__ block_tables,
                                                              const int* __restrict__ token_seq,
                                                              const int* __restrict__ token_pos, int64_t tokens,
                                                              int block_size, int max_blocks) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  constexpr int KEEP = 4;                              // register steps: rank up to 32 * VEC * KEEP stays in registers
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int seq = token_seq[t], pos = token_pos[t];
  const int64_t row = (int64_t)block_tables[(int64_t)seq * max_blocks + pos / block_size] * block_size + pos % block_size;
  const T* zr = z + t * ldz;
  T* out = cache + row * (rank + rot);
  Pack keep[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int n = 0; n < KEEP; ++n) {
    const int i = (lane + 32 * n) * VEC;
    if (i < rank) {
      keep[n] = *reinterpret_cast<const Pack*>(zr + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) { const float v = to_f32<T>(keep[n].v[e]); ss = fmaf(v, v, ss); }
    }
  }
  for (int i = (lane + 32 * KEEP) * VEC; i < rank; i += 32 * VEC) {
    const Pack a = *reinterpret_cast<const Pack*>(zr + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) { const float v = to_f32<T>(a.v[e]); ss = fmaf(v, v, ss); }
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)rank + eps);
  auto emit = [&](int i, const Pack& a) {
    Pack o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) o.v[e] = from_f32<T>(to_f32<T>(a.v[e]) * r * to_f32<TW>(w[i + e]));
    *reinterpret_cast<Pack*>(out + i) = o;
  };
#pragma unroll
  for (int n = 0; n < KEEP; ++n) {
    const int i = (lane + 32 * n) * VEC;
    if (i < rank) emit(i, keep[n]);
  }
  for (int i = (lane + 32 * KEEP) * VEC; i < rank; i += 32 * VEC) emit(i, *reinterpret_cast<const Pack*>(zr + i));
  const int half = rot >> 1;
  const float* cs = table + (int64_t)pos * rot;
  for (int i = lane; i < half; i += 32) {
    const float u = to_f32<T>(zr[rank + i]), v = to_f32<T>(zr[rank + half + i]);
    const float c = cs[i], sn = cs[half + i];
    out[rank + i] = from_f32<T>(u * c - v * sn);
    out[rank + half + i] = from_f32<T>(v * c + u * sn);
  }
}

// ------------------------------------------------------------------------------------------------ clamped gated unit
// gu [rows, 2 I] = gate | up.  IEEE fp32 arithmetic (this file is built without fast math), one rounding into T.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int I,
                                                          float limit, float alpha, const int64_t* __restrict__ row_limit) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  if (row_limit != nullptr) rows = min(rows, *row_limit);
  const int per_row = I / VEC;
  const int64_t total = rows * per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / per_row;
    const int c = (int)(idx - r * per_row) * VEC;
    const Pack gp = *reinterpret_cast<const Pack*>(gu + r * 2 * I + c);
    const Pack up = *reinterpret_cast<const Pack*>(gu + r * 2 * I + I + c);
    Pack o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float gq = fminf(to_f32<T>(gp.v[e]), limit);
      const float u = fminf(fmaxf(to_f32<T>(up.v[e]), -limit), limit);
      o.v[e] = from_f32<T>(gq * sigmoid_f(alpha * gq) * (u + 1.f));
    }
    *reinterpret_cast<Pack*>(out + r * I + c) = o;
  }
}

// ------------------------------------------------------------------------------------------------ paged cache write
template <typename T>
__global__ void __launch_bounds__(128) paged_kv_write_mix_kernel(const T* __restrict__ k, int64_t ldk, const T* __restrict__ v,
                                                                 int64_t ldv, const T* __restrict__ v_other,
                                                                 int64_t ldvo, float lam, T* __restrict__ k_cache,
                                                                 T* __restrict__ v_cache,
                                                                 const int* __restrict__ block_tables,
                                                                 const int* __restrict__ token_seq,
                                                                 const int* __restrict__ token_pos, int kw, int vw,
                                                                 int block_size, int max_blocks) {
  const int64_t t = blockIdx.x;
  const int seq = token_seq[t], pos = token_pos[t];
  const int64_t row = (int64_t)block_tables[(int64_t)seq * max_blocks + pos / block_size] * block_size + pos % block_size;
  for (int i = threadIdx.x; i < kw; i += blockDim.x) k_cache[row * kw + i] = k[t * ldk + i];
  for (int i = threadIdx.x; i < vw; i += blockDim.x) {
    T val = v[t * ldv + i];
    if (v_other != nullptr)
      val = from_f32<T>((1.f - lam) * to_f32<T>(val) + lam * to_f32<T>(v_other[t * ldvo + i]));
    v_cache[row * vw + i] = val;
  }
}

// ------------------------------------------------------------------------------------------------ paged attention
// One warp per (step token, query head).  Keys 0..pos of the token's sequence are walked in tiles of 32 in a fixed order
// (lane = key for the scores, lane = value channel for the weighted sum), online softmax in fp32.  With `sink` the running
// maximum starts at the sink's score (`sink_vals[head]`, 0 without the table) and the denominator at 1: a key of that
// score without a value, not scaled.  `slopes[head]` takes slope * (pos - key) off every score; `window` > 0 keeps the
// keys pos - window + 1 .. pos only.
constexpr int ATT_MAX_VREG = 16;  // value width up to 512

template <typename T>
__global__ void __launch_bounds__(128) paged_bias_attention_kernel(
    const T* __restrict__ q, int64_t ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
    const float* __restrict__ bias_table, const int* __restrict__ bucket_start, int nbuckets, T* __restrict__ out,
    int64_t tokens, int heads, int kv_heads, int dim, int vdim, int ldv, int block_size, int max_blocks, float scale,
    int sink, int mask_block, const float* __restrict__ sink_vals, const float* __restrict__ slopes, int window) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* qs = smem + warp * dim;
  int* bstart = reinterpret_cast<int*>(smem + nwarps * dim);
  for (int i = threadIdx.x; i < nbuckets; i += blockDim.x) bstart[i] = bucket_start[i];
  const int64_t unit = (int64_t)blockIdx.x * nwarps + warp;
  const bool live = unit < tokens * heads;
  const int64_t t = live ? unit / heads : 0;
  const int h = live ? (int)(unit % heads) : 0;
  for (int i = lane; i < dim; i += 32) qs[i] = live ? to_f32<T>(q[t * ldq + h * dim + i]) * scale : 0.f;
  __syncthreads();
  if (!live) return;
  const int g = h / (heads / kv_heads);
  const int seq = token_seq[t], pos = token_pos[t];
  const int* bt = block_tables + (int64_t)seq * max_blocks;
  const int half = nbuckets >> 1;
  float m = sink ? (sink_vals != nullptr ? sink_vals[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;
  const float slope = slopes != nullptr ? slopes[h] : 0.f;
  float acc[ATT_MAX_VREG];
#pragma unroll
  for (int r = 0; r < ATT_MAX_VREG; ++r) acc[r] = 0.f;
  // with a block mask the keys start at the first position of the query's own block, with a window at its first key
  int jfirst = mask_block > 0 ? pos / mask_block * mask_block : 0;
  if (window > 0) jfirst = max(jfirst, pos - window + 1);
  for (int j0 = jfirst; j0 <= pos; j0 += 32) {
    const int jk = j0 + lane;
    float sc = -INFINITY;
    int64_t myrow = 0;
    if (jk <= pos) {
      myrow = ((int64_t)bt[jk / block_size] * block_size + jk % block_size) * kv_heads + g;
      const T* kr = k_cache + myrow * dim;
      float d0 = 0.f, d1 = 0.f;
      int i = 0;
      for (; i + 1 < dim; i += 2) {
        d0 = fmaf(qs[i], to_f32<T>(kr[i]), d0);
        d1 = fmaf(qs[i + 1], to_f32<T>(kr[i + 1]), d1);
      }
      if (i < dim) d0 = fmaf(qs[i], to_f32<T>(kr[i]), d0);
      sc = d0 + d1;
      if (nbuckets > 0) {
        const int n = pos - jk;
        int b = n;
        if (n >= half) {
          b = half;
          while (b + 1 < nbuckets && bstart[b + 1] <= n) ++b;
        }
        sc += bias_table[b * heads + h];
      }
      sc -= slope * (float)(pos - jk);
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float alpha = expf(m - mn);           // m = -inf only before the first tile without a sink: exp(-inf) = 0
    const float pj = jk <= pos ? expf(sc - mn) : 0.f;
    l = l * alpha + warp_sum(pj);
    m = mn;
#pragma unroll
    for (int r = 0; r < ATT_MAX_VREG; ++r) acc[r] *= alpha;
    const int nk = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const int64_t vrow = __shfl_sync(0xffffffffu, myrow, jj);
      const T* vr = v_cache + vrow * ldv;      // ldv = vdim, or the key row's width when the values live in the key rows
#pragma unroll
      for (int r = 0; r < ATT_MAX_VREG; ++r) {
        const int c = lane + 32 * r;
        if (c < vdim) acc[r] = fmaf(pw, to_f32<T>(vr[c]), acc[r]);
      }
    }
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int r = 0; r < ATT_MAX_VREG; ++r) {
    const int c = lane + 32 * r;
    if (c < vdim) out[t * ((int64_t)heads * vdim) + h * vdim + c] = from_f32<T>(acc[r] * inv);
  }
}

// ------------------------------------------------------------------------------------------------ tensor-core variant
// 16-bit inputs: a CTA of 4 warps owns 64 query ROWS of one (sequence, kv head): row = (token of the portion, query head
// of the kv head's group), so the K / V tile that cp.async brings from the pages is shared by the whole group and a
// decoded token fills rows with its group's heads.  S = Q K^T and O += P V run on mma.sync m16n8k16 with fp32
// accumulators; softmax, bias and sink in fp32 registers.  D = head width rounded up (zero padded in shared memory).
constexpr int MMA_BM = 64, MMA_BN = 64;

template <typename T> CB_DEVICE void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> CB_DEVICE void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> CB_DEVICE void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> CB_DEVICE uint32_t pack2(float lo, float hi);
template <> CB_DEVICE uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> CB_DEVICE uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// what a pair of fp32 values loses when it is packed into 16 bits: the second operand of a two-term product
template <typename T> CB_DEVICE uint32_t pack2_rest(float lo, float hi, uint32_t packed);
template <> CB_DEVICE uint32_t pack2_rest<__nv_bfloat16>(float lo, float hi, uint32_t packed) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  return pack2<__nv_bfloat16>(lo - f.x, hi - f.y);
}
template <> CB_DEVICE uint32_t pack2_rest<__half>(float lo, float hi, uint32_t packed) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&packed));
  return pack2<__half>(lo - f.x, hi - f.y);
}
CB_DEVICE float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
CB_DEVICE void cp_async16(void* smem_dst, const void* gmem_src, uint32_t src_bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}

// Key range split (decode steps, few CTAs): with `chunk` > 0 grid.x also enumerates key chunks; a CTA then writes its
// unnormalised partial (fp32 accumulator, running maximum, denominator without the sink) and `attention_merge_kernel`
// joins the chunks of every (token, head) in ascending order.
//
// A CTA is 4 warps x 32 rows (MT = 2 m16 tiles per warp) when a portion fills 128 rows, 4 x 16 (MT = 1) otherwise.  Two
// m-tiles per warp halve the shared-memory reads per MMA (a K / V fragment feeds both) and double the independent
// accumulator chains.  The query tile sits in shared memory (A fragments by ldmatrix.x4, K fragments by ldmatrix.x4
// for two k-steps at once, V fragments by ldmatrix.x2.trans).
CB_DEVICE void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

//
// KS (decode steps: every sequence of the launch brings at most 16 rows = one m16 tile): the four warps share the SAME 16
// rows and split each key tile between them (16 keys per warp) instead of three of them idling; every warp keeps its own
// running maximum, denominator and accumulator, and the four are joined through shared memory at the end.
template <typename T, int D, int MT, bool KS>
__global__ void __launch_bounds__(128, D > 128 ? 1 : (MT == 2 ? 2 : 3)) paged_bias_attention_mma_kernel(
    const T* __restrict__ q, int64_t ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_tables, const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const float* __restrict__ bias_table, const uint8_t* __restrict__ lut, int lut_n, int nbuckets, T* __restrict__ out,
    int heads, int kv_heads, int dim, int vdim, int ldv, int block_size, int max_blocks, float scale, int sink, int chunk,
    int max_splits, float* __restrict__ part_o, float* __restrict__ part_ml, int mask_block, int wide_weights,
    const float* __restrict__ sink_vals, const float* __restrict__ slopes, int window) {
  constexpr int BM = 64 * MT;
  constexpr int LDS = D + 8;                    // padded row: 16-byte aligned, conflict-free fragment reads
  constexpr int TILE = MMA_BN * LDS;
  constexpr int NR = 2 * MT;                    // rows a thread owns: (m-tile, upper / lower half)
  constexpr int NT = KS ? 2 : MMA_BN / 8;       // n8 key tiles a warp scores per key tile
  constexpr int KK = KS ? 1 : MMA_BN / 16;      // k16 steps of its P V product
  static_assert(!KS || MT == 1, "the key-splitting form holds one m16 tile");
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // values that live in the key rows (latent attention: value = the row's first vdim columns): the K tile serves as V
  const bool kv_same = v_cache == k_cache && ldv == dim;
  const int stage_elems = kv_same ? TILE : 2 * TILE;
  T* KV = reinterpret_cast<T*>(smem_raw);       // [2 stages][K tile | V tile] (no V tile when the K tile serves as V)
  T* Qs = KV + 2 * stage_elems;                 // [BM][LDS]
  float* tab = reinterpret_cast<float*>(Qs + BM * LDS);              // [nbuckets][R] of this kv head's group
  const int s = blockIdx.z, g = blockIdx.y;
  const int R = heads / kv_heads;
  const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
  const int split = chunk > 0 ? blockIdx.x % max_splits : 0;
  const int nrows = qlen * R, row0 = (chunk > 0 ? blockIdx.x / max_splits : blockIdx.x) * BM;
  if (row0 >= nrows) return;
  const int ctx = ctx_len[s];
  const int last_row = min(nrows - 1, row0 + BM - 1);
  // block mask: a row at position p sees keys p / mask_block * mask_block .. p; the tile's keys start at its first row's
  // block (key chunks that end below it are never read: the merge starts at the row's own first chunk)
  // (rounded down to a key tile, so that tiles keep their place inside a key chunk and never reach into the next one)
  // A window of `window` positions moves a row's first key to pos - window + 1 in the same way (both grow with pos).
  auto first_key = [&](int p) {
    int f = mask_block > 0 ? p / mask_block * mask_block : 0;
    if (window > 0) f = max(f, p - window + 1);
    return f;
  };
  const bool masked_lo = mask_block > 0 || window > 0;
  const int blk_lo = masked_lo ? first_key(ctx + row0 / R) / MMA_BN * MMA_BN : 0;
  const int key_lo = max(chunk > 0 ? split * chunk : 0, blk_lo);
  const int pos_max = chunk > 0 ? min(ctx + last_row / R, split * chunk + chunk - 1) : ctx + last_row / R;
  if (key_lo > pos_max) return;                 // this chunk lies beyond (or below) every row of the tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  for (int i = tid; i < nbuckets * R; i += 128) tab[i] = bias_table[(i / R) * heads + g * R + (i % R)] * LOG2E;
  const int* bt = block_tables + (int64_t)s * max_blocks;

  auto load_tile = [&](int stage, int j0) {
    constexpr int CH = D / 8;
    T* Ks = KV + stage * stage_elems;
    T* Vs = Ks + TILE;
    for (int idx = tid; idx < MMA_BN * CH; idx += 128) {
      const int r = idx / CH, c8 = (idx % CH) * 8;
      const int j = j0 + r;
      const bool in = j <= pos_max;
      const int64_t row = in ? ((int64_t)bt[j / block_size] * block_size + j % block_size) * kv_heads + g : 0;
      const bool kin = in && c8 < dim, vin = in && c8 < vdim;
      cp_async16(Ks + r * LDS + c8, k_cache + (kin ? row * dim + c8 : 0), kin ? 16u : 0u);
      if (!kv_same) cp_async16(Vs + r * LDS + c8, v_cache + (vin ? row * ldv + c8 : 0), vin ? 16u : 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  {                                             // the query tile rides in the first copy group
    constexpr int CH = D / 8;
    for (int idx = tid; idx < BM * CH; idx += 128) {
      const int r = idx / CH, c8 = (idx % CH) * 8;
      const int row = row0 + r;
      const bool in = row < nrows && c8 < dim;
      cp_async16(Qs + r * LDS + c8, q + (in ? (int64_t)(t0 + row / R) * ldq + (g * R + row % R) * dim + c8 : 0),
                 in ? 16u : 0u);
    }
  }
  load_tile(0, key_lo);

  int rr[NR], pos[NR], hr[NR], lo[NR];
  bool valid[NR];
#pragma unroll
  for (int e = 0; e < NR; ++e) {
    rr[e] = row0 + (KS ? 0 : warp * (16 * MT)) + (e >> 1) * 16 + gid + 8 * (e & 1);
    valid[e] = rr[e] < nrows;
    hr[e] = valid[e] ? rr[e] % R : 0;
    pos[e] = valid[e] ? ctx + rr[e] / R : -1;
    lo[e] = (masked_lo && valid[e]) ? first_key(pos[e]) : 0;      // first key the row sees
  }
  float o[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nv = 0; nv < D / 8; ++nv)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][nv][e] = 0.f;
  float m[NR], l[NR], sk[NR], sl[NR], slb[NR];
#pragma unroll
  for (int e = 0; e < NR; ++e) {
    sk[e] = (sink_vals != nullptr && valid[e]) ? sink_vals[g * R + hr[e]] * LOG2E : 0.f;      // the sink's score
    sl[e] = (slopes != nullptr && valid[e]) ? slopes[g * R + hr[e]] * LOG2E : 0.f;            // score -= sl * (pos - key)
    slb[e] = -sl[e] * (float)pos[e];
    m[e] = (sink && chunk == 0) ? sk[e] : -INFINITY;        // log2 domain; with chunks the sink joins in the merge
    l[e] = 0.f;                                 // per-thread partial; the sink's share is added once at the end
  }
  const float sc2 = scale * LOG2E;
  // first / last position any row of this warp sees: tiles beyond are skipped, tiles before need no causal test
  const int wrow0 = row0 + (KS ? 0 : warp * (16 * MT));
  const int koff = KS ? warp * 16 : 0;          // first key of the warp inside a key tile
  const bool wlive = wrow0 < nrows;
  const int wlo = ctx + min(nrows - 1, wrow0) / R;
  const int whi = wlive ? ctx + min(nrows - 1, wrow0 + 16 * MT - 1) / R : -1;
  const int wblk = (masked_lo && wlive) ? first_key(whi) : 0;     // latest first key among its rows
  const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + ((KS ? 0 : warp * 16 * MT) + (lane & 15)) * LDS +
                                                             (lane >> 4) * 8);

  int stage = 0;
  for (int j0 = key_lo; j0 <= pos_max; j0 += MMA_BN, stage ^= 1) {
    if (j0 + MMA_BN <= pos_max) {               // the other stage was released by the barrier that ended the last pass
      load_tile(stage ^ 1, j0 + MMA_BN);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (j0 + koff <= whi) {                     // warp-uniform: otherwise the whole tile is masked for this warp
      const T* Ks = KV + stage * stage_elems;
      const T* Vs = kv_same ? Ks : Ks + TILE;
      float sacc[MT][NT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) sacc[mt][nt][e] = 0.f;
      const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Ks + (koff + (lane & 7)) * LDS + (lane >> 3) * 8);
#pragma unroll
      for (int kp = 0; kp < D / 32; ++kp) {     // two k-steps of 16 per pass
        uint32_t qa[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          ldsm_x4(qa[mt][0], q_addr + (mt * 16 * LDS + kp * 32) * (uint32_t)sizeof(T));
          ldsm_x4(qa[mt][1], q_addr + (mt * 16 * LDS + kp * 32 + 16) * (uint32_t)sizeof(T));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t kb[4];
          ldsm_x4(kb, k_addr + (nt * 8 * LDS + kp * 32) * (uint32_t)sizeof(T));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<T>(sacc[mt][nt], qa[mt][0], kb[0], kb[1]);
            mma_16816<T>(sacc[mt][nt], qa[mt][1], kb[2], kb[3]);
          }
        }
      }
      const int jlast = j0 + koff + NT * 8 - 1;  // last key this warp scores in the tile
      const bool unmasked = jlast <= wlo && j0 + koff >= wblk;
      const bool far = nbuckets == 0 || wlo - jlast >= lut_n;                 // every distance in the last bucket
      float fb[NR];
#pragma unroll
      for (int e = 0; e < NR; ++e) fb[e] = nbuckets > 0 ? tab[(nbuckets - 1) * R + hr[e]] : 0.f;
      float mx[NR];
#pragma unroll
      for (int e = 0; e < NR; ++e) mx[e] = m[e];
      if (unmasked && far) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = mt * 2 + (e >> 1);
              float sv = fmaf(sacc[mt][nt][e], sc2, fb[r]);
              if (slopes != nullptr) sv += fmaf(sl[r], (float)(j0 + koff + nt * 8 + tig * 2 + (e & 1)), slb[r]);
              sacc[mt][nt][e] = sv;
              mx[r] = fmaxf(mx[r], sv);
            }
      } else {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = mt * 2 + (e >> 1), j = j0 + koff + nt * 8 + tig * 2 + (e & 1);
              float sv = -INFINITY;
              if (j <= pos[r] && j >= lo[r]) {
                sv = sacc[mt][nt][e] * sc2;
                if (nbuckets > 0) {
                  const int n = pos[r] - j;
                  sv += n < lut_n ? tab[(int)__ldg(lut + n) * R + hr[r]] : fb[r];
                }
                if (slopes != nullptr) sv += fmaf(sl[r], (float)j, slb[r]);
              }
              sacc[mt][nt][e] = sv;
              mx[r] = fmaxf(mx[r], sv);
            }
      }
      float alpha[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mu = mx[r] == -INFINITY ? 0.f : mx[r];
        alpha[r] = ex2f(m[r] - mu);             // m = -inf -> 0
        m[r] = mx[r];
        l[r] *= alpha[r];
        mx[r] = mu;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nv = 0; nv < D / 8; ++nv) {
          o[mt][nv][0] *= alpha[mt * 2]; o[mt][nv][1] *= alpha[mt * 2];
          o[mt][nv][2] *= alpha[mt * 2 + 1]; o[mt][nv][3] *= alpha[mt * 2 + 1];
        }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = mt * 2 + (e >> 1);
            const float pe = ex2f(sacc[mt][nt][e] - mx[r]);
            sacc[mt][nt][e] = pe;
            l[r] += pe;
          }
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        uint32_t pa[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          pa[mt][0] = pack2<T>(sacc[mt][2 * kk][0], sacc[mt][2 * kk][1]);
          pa[mt][1] = pack2<T>(sacc[mt][2 * kk][2], sacc[mt][2 * kk][3]);
          pa[mt][2] = pack2<T>(sacc[mt][2 * kk + 1][0], sacc[mt][2 * kk + 1][1]);
          pa[mt][3] = pack2<T>(sacc[mt][2 * kk + 1][2], sacc[mt][2 * kk + 1][3]);
        }
        // `wide_weights`: the softmax weights enter P V as a 16-bit value plus the 16-bit rest of its rounding (two MMAs
        // per fragment), so a weight keeps about 16 bits of mantissa instead of 8
        uint32_t pr[MT][4];
        if (wide_weights) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            pr[mt][0] = pack2_rest<T>(sacc[mt][2 * kk][0], sacc[mt][2 * kk][1], pa[mt][0]);
            pr[mt][1] = pack2_rest<T>(sacc[mt][2 * kk][2], sacc[mt][2 * kk][3], pa[mt][1]);
            pr[mt][2] = pack2_rest<T>(sacc[mt][2 * kk + 1][0], sacc[mt][2 * kk + 1][1], pa[mt][2]);
            pr[mt][3] = pack2_rest<T>(sacc[mt][2 * kk + 1][2], sacc[mt][2 * kk + 1][3], pa[mt][3]);
          }
        }
        const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(Vs + (koff + kk * 16 + (lane & 15)) * LDS);
#pragma unroll
        for (int nv = 0; nv < D / 8; ++nv) {
          uint32_t b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                       : "=r"(b0), "=r"(b1) : "r"(vrow + nv * 16));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_16816<T>(o[mt][nv], pa[mt], b0, b1);
          if (wide_weights) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_16816<T>(o[mt][nv], pr[mt], b0, b1);
          }
        }
      }
    }
    __syncthreads();                            // this stage may be refilled in the next pass
  }
  if (KS) {
    // the four warps' partial (maximum, denominator, accumulator) of the shared 16 rows meet in shared memory (the key
    // loop's last barrier has released the K / V stages) and every thread joins a share of the (row, column) pairs
    float* mg = reinterpret_cast<float*>(smem_raw);          // [4 warps][16 rows][D + 2]: columns, then m, l
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      float* base = mg + (warp * 16 + gid + 8 * r) * (D + 2);
#pragma unroll
      for (int nv = 0; nv < D / 8; ++nv) {
        base[nv * 8 + tig * 2] = o[0][nv][2 * r];
        base[nv * 8 + tig * 2 + 1] = o[0][nv][2 * r + 1];
      }
      if (tig == 0) { base[D] = m[r]; base[D + 1] = l[r]; }
    }
    __syncthreads();
    for (int e = tid; e < 16 * vdim; e += 128) {
      const int rl = e / vdim, c = e - rl * vdim;
      const int row = row0 + rl;
      if (row >= nrows) break;
      float mw[4], mall = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) { mw[w] = mg[(w * 16 + rl) * (D + 2) + D]; mall = fmaxf(mall, mw[w]); }
      const float mu = mall == -INFINITY ? 0.f : mall;
      float lsum = 0.f, osum = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = ex2f(mw[w] - mu);                     // m = -inf (no key seen) -> 0
        lsum = fmaf(mg[(w * 16 + rl) * (D + 2) + D + 1], f, lsum);
        osum = fmaf(mg[(w * 16 + rl) * (D + 2) + c], f, osum);
      }
      const int64_t unit = (int64_t)(t0 + row / R) * heads + g * R + row % R;
      if (chunk > 0) {
        part_o[(unit * max_splits + split) * vdim + c] = osum;
        if (c == 0) {
          part_ml[(unit * max_splits + split) * 2] = mall;
          part_ml[(unit * max_splits + split) * 2 + 1] = lsum;
        }
      } else {
        if (sink) lsum += ex2f((sink_vals != nullptr ? sink_vals[g * R + row % R] * LOG2E : 0.f) - mu);
        out[unit * vdim + c] = from_f32<T>(lsum > 0.f ? osum / lsum : 0.f);
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    if (!valid[r]) continue;
    const int mt = r >> 1, hf = r & 1;
    const int64_t unit = (int64_t)(t0 + rr[r] / R) * heads + g * R + hr[r];
    if (chunk > 0) {
      float* po = part_o + (unit * max_splits + split) * vdim;
      if (tig == 0) {
        part_ml[(unit * max_splits + split) * 2] = m[r];
        part_ml[(unit * max_splits + split) * 2 + 1] = l[r];
      }
#pragma unroll
      for (int nv = 0; nv < D / 8; ++nv) {
        const int c = nv * 8 + tig * 2;
        if (c < vdim) *reinterpret_cast<float2*>(po + c) = make_float2(o[mt][nv][2 * hf], o[mt][nv][2 * hf + 1]);
      }
      continue;
    }
    if (sink) l[r] += ex2f(sk[r] - (m[r] == -INFINITY ? 0.f : m[r]));
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    T* orow = out + unit * vdim;
#pragma unroll
    for (int nv = 0; nv < D / 8; ++nv) {
      const int c = nv * 8 + tig * 2;
      if (c < vdim)
        *reinterpret_cast<uint32_t*>(orow + c) = pack2<T>(o[mt][nv][2 * hf] * inv, o[mt][nv][2 * hf + 1] * inv);
    }
  }
}

// one warp per (token, head, 32 value columns): joins the key chunks 0..pos / chunk (log2-domain maxima).  The chunks'
// maxima and denominators are read with one chunk per lane and reduced over the warp; the weighted sum of the partial
// outputs then walks the chunks in ascending order with the weights passed by shuffle, eight chunks' loads in flight.
template <typename T>
__global__ void __launch_bounds__(128) attention_merge_kernel(const float* __restrict__ part_o,
                                                              const float* __restrict__ part_ml,
                                                              const int* __restrict__ token_pos, T* __restrict__ out,
                                                              int64_t tokens, int heads, int vdim, int chunk,
                                                              int max_splits, int sink, int mask_block,
                                                              const float* __restrict__ sink_vals, int window) {
  const int lane = threadIdx.x & 31;
  const int cblocks = (vdim + 31) >> 5;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= tokens * heads * cblocks) return;
  const int64_t unit = item / cblocks;
  const int c = (int)(item % cblocks) * 32 + lane;
  const int tpos = token_pos[unit / heads];
  const int nsp = tpos / chunk + 1;
  int kfirst = mask_block > 0 ? tpos / mask_block * mask_block : 0;
  if (window > 0) kfirst = max(kfirst, tpos - window + 1);
  const int sp0 = kfirst / chunk;                                                     // first chunk with a visible key
  const float* ml = part_ml + unit * max_splits * 2;
  const float sk = sink_vals != nullptr ? sink_vals[unit % heads] * 1.4426950408889634f : 0.f;
  float mm = sink ? sk : -INFINITY;
  for (int sp = sp0 + lane; sp < nsp; sp += 32) mm = fmaxf(mm, ml[sp * 2]);
  mm = warp_max(mm);
  const float mu = mm == -INFINITY ? 0.f : mm;
  float l = 0.f;
  for (int sp = sp0 + lane; sp < nsp; sp += 32) l = fmaf(ml[sp * 2 + 1], ex2f(ml[sp * 2] - mu), l);
  l = warp_sum(l) + (sink ? ex2f(sk - mu) : 0.f);
  float acc = 0.f;
  const float* po = part_o + unit * max_splits * vdim;
  for (int s0 = sp0; s0 < nsp; s0 += 32) {
    const float wl = s0 + lane < nsp ? ex2f(ml[(s0 + lane) * 2] - mu) : 0.f;      // weight of chunk s0 + lane
    const int n = min(32, nsp - s0);
#pragma unroll 8
    for (int j = 0; j < n; ++j) {
      const float w = __shfl_sync(0xffffffffu, wl, j);
      if (c < vdim) acc = fmaf(po[(int64_t)(s0 + j) * vdim + c], w, acc);
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  if (c < vdim) out[unit * vdim + c] = from_f32<T>(acc * inv);
}

template <typename T, int D, int MT, bool KS = false>
int launch_attention_mma(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* cu_q, const int* ctx_len, const int* token_pos, const float* bias_table,
                         const uint8_t* lut, int lut_n, int nbuckets, void* out, int64_t tokens, int nseq, int max_q,
                         int heads, int kv_heads, int dim, int vdim, int ldv, int block_size, int max_blocks, float scale,
                         int sink, int chunk, int max_splits, float* part_o, float* part_ml, int mask_block,
                         int wide_weights, const float* sink_vals, const float* slopes, int window, cudaStream_t st) {
  const int R = heads / kv_heads;
  constexpr int BM = 64 * MT;
  const bool kv_same = v_cache == k_cache && ldv == dim;
  const size_t smem = (size_t)((kv_same ? 2 : 4) * MMA_BN + BM) * (D + 8) * sizeof(T) + (size_t)nbuckets * R * sizeof(float);
  auto kern = paged_bias_attention_mma_kernel<T, D, MT, KS>;
  static bool configured = false;               // per instantiation: opt in to large shared memory, all of it for CTAs
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int rowtiles = (max_q * R + BM - 1) / BM;
  dim3 grid(rowtiles * (chunk > 0 ? max_splits : 1), kv_heads, nseq);
  kern<<<grid, 128, smem, st>>>((const T*)q, ldq, (const T*)k_cache, (const T*)v_cache, block_tables, cu_q, ctx_len,
                                bias_table, lut, lut_n, nbuckets, (T*)out, heads, kv_heads, dim, vdim, ldv, block_size,
                                max_blocks, scale, sink, chunk, max_splits, part_o, part_ml, mask_block, wide_weights,
                                sink_vals, slopes, window);
  if (chunk > 0) {
    const int64_t units = tokens * heads * ((vdim + 31) / 32);
    attention_merge_kernel<T><<<(unsigned)((units + 3) / 4), 128, 0, st>>>(part_o, part_ml, token_pos, (T*)out, tokens,
                                                                          heads, vdim, chunk, max_splits, sink, mask_block,
                                                                          sink_vals, window);
  }
  return CB_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------------ gated linear recurrence
// One thread per (sequence, channel): S <- a_t S + sqrt(1 - a_t^2) i_t u_t over the portion's tokens, out = S gelu_tanh(y).
// r = sigmoid(gate_r + bias), i = sigmoid(gate_i + bias), log a = -c r softplus(lam); 1 - a^2 = -expm1(2 log a) keeps its
// digits when a is close to one.  gates [blocks, T, 2 bw] fp32: channel j of block b at [b][t][j] (recurrence gate) and
// [b][t][bw + j] (input gate).  Everything that does not depend on S - loads, gates, the branch - is done for LRU_UNROLL
// tokens at once, so their loads are in flight together; the chain through S is one FMA per token.
constexpr int LRU_UNROLL = 8;

template <typename T>
__global__ void __launch_bounds__(128) lru_scan_kernel(const T* __restrict__ u, int64_t ldu, const float* __restrict__ gates,
                                                       const float* __restrict__ gbias, const float* __restrict__ lam,
                                                       const T* __restrict__ branch, int64_t ldb, float* __restrict__ state,
                                                       T* __restrict__ out, int64_t tokens, const int* __restrict__ cu_q,
                                                       const int* __restrict__ ctx_len, const int* __restrict__ slots,
                                                       int C, int nb, float cmul) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  const int t0 = cu_q[s], t1 = cu_q[s + 1];
  if (c >= C || t0 >= t1) return;
  const int bw = C / nb, b = c / bw, j = c % bw;
  const float br = gbias[(int64_t)b * 2 * bw + j], bi = gbias[(int64_t)b * 2 * bw + bw + j];
  const float cl = -cmul * softplus_f(lam[c]);
  float* Sg = state + (int64_t)slots[s] * C + c;
  float S = ctx_len[s] > 0 ? *Sg : 0.f;
  const float* gp = gates + (int64_t)b * tokens * 2 * bw + j;
  for (int tb = t0; tb < t1; tb += LRU_UNROLL) {
    float gr[LRU_UNROLL], gi[LRU_UNROLL], uu[LRU_UNROLL], yy[LRU_UNROLL];
#pragma unroll
    for (int e = 0; e < LRU_UNROLL; ++e) {
      const int64_t t = min(tb + e, t1 - 1);
      gr[e] = gp[t * 2 * bw];
      gi[e] = gp[t * 2 * bw + bw];
      uu[e] = to_f32<T>(u[t * ldu + c]);
      yy[e] = to_f32<T>(branch[t * ldb + c]);
    }
    float a[LRU_UNROLL], x[LRU_UNROLL];
#pragma unroll
    for (int e = 0; e < LRU_UNROLL; ++e) {
      const float la = cl * sigmoid_f(gr[e] + br);
      a[e] = expf(la);
      x[e] = sqrtf(-expm1f(2.f * la)) * sigmoid_f(gi[e] + bi) * uu[e];
      yy[e] = gelu_tanh_f(yy[e]);
    }
#pragma unroll
    for (int e = 0; e < LRU_UNROLL; ++e) {
      if (tb + e < t1) {
        S = fmaf(a[e], S, x[e]);
        out[(int64_t)(tb + e) * C + c] = from_f32<T>(S * yy[e]);
      }
    }
  }
  *Sg = S;
}

// ------------------------------------------------------------------------------------------------ rotary + unit norm
// One warp per (token, head), in place: the head's first rot_dims channels are turned by the token's position (table row
// = cos | sin of rot_dims / 2 angles; pairs (2i, 2i + 1) when interleaved, else (i, i + rot_dims / 2)), then, with
// `unit`, the whole head is divided by sqrt(mean of squares + eps).  The head sits in shared memory while it is turned.
constexpr int ROT_MAX_REG = 16;        // head width up to 512

template <typename T>
__global__ void __launch_bounds__(128) rotary_unit_norm_kernel(T* __restrict__ x, int64_t ldx, int64_t tokens, int heads,
                                                               int dim, int rot_dims, int interleaved,
                                                               const float* __restrict__ table,
                                                               const int* __restrict__ token_pos, int unit, float eps) {
  extern __shared__ float rot_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= tokens * heads) return;
  const int64_t t = item / heads;
  const int h = (int)(item % heads);
  T* row = x + t * ldx + (int64_t)h * dim;
  float* sm = rot_smem + warp * dim;
  for (int i = lane; i < dim; i += 32) sm[i] = to_f32<T>(row[i]);
  __syncwarp();
  const int half = rot_dims >> 1;
  const float* cs = rot_dims > 0 ? table + (int64_t)token_pos[t] * rot_dims : nullptr;
  float y[ROT_MAX_REG];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < ROT_MAX_REG; ++e) {
    const int c = lane + 32 * e;
    y[e] = 0.f;
    if (c < dim) {
      float v = sm[c];
      if (c < rot_dims) {
        if (interleaved) {
          const float cc = cs[c >> 1], sn = cs[half + (c >> 1)];
          v = (c & 1) ? sm[c] * cc + sm[c - 1] * sn : sm[c] * cc - sm[c + 1] * sn;
        } else if (c < half) {
          v = sm[c] * cs[c] - sm[c + half] * cs[half + c];
        } else {
          v = sm[c] * cs[c - half] + sm[c - half] * cs[c];
        }
      }
      y[e] = v;
      ss = fmaf(v, v, ss);
    }
  }
  float r = 1.f;
  if (unit) r = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
#pragma unroll
  for (int e = 0; e < ROT_MAX_REG; ++e) {
    const int c = lane + 32 * e;
    if (c < dim) row[c] = from_f32<T>(y[e] * r);
  }
}

// Interleaved pairs sit side by side, so a lane that holds four adjacent channels turns two whole pairs by itself: no
// staging, 8-byte (16-bit types) or 16-byte (fp32) accesses.  One warp per (token, head); head widths up to 512 that
// are multiples of 4, rot_dims a multiple of 4 too (the launcher checks, alignment included).
template <typename T>
__global__ void __launch_bounds__(128) rotary_pairs_unit_norm_kernel(T* __restrict__ x, int64_t ldx, int64_t tokens,
                                                                     int heads, int dim, int rot_dims,
                                                                     const float* __restrict__ table,
                                                                     const int* __restrict__ token_pos, int unit,
                                                                     float eps) {
  struct alignas(sizeof(T) * 4) Pack { T v[4]; };
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= tokens * heads) return;
  const int64_t t = item / heads;
  T* row = x + t * ldx + (int64_t)(item % heads) * dim;
  const int half = rot_dims >> 1;
  const float* cs = rot_dims > 0 ? table + (int64_t)token_pos[t] * rot_dims : nullptr;
  float y[4][4];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = (lane + 32 * e) * 4;
    if (c < dim) {
      const Pack a = *reinterpret_cast<const Pack*>(row + c);
      float v0 = to_f32<T>(a.v[0]), v1 = to_f32<T>(a.v[1]), v2 = to_f32<T>(a.v[2]), v3 = to_f32<T>(a.v[3]);
      if (c < rot_dims) {
        const float2 cc = *reinterpret_cast<const float2*>(cs + (c >> 1));
        const float2 sn = *reinterpret_cast<const float2*>(cs + half + (c >> 1));
        const float r0 = v0 * cc.x - v1 * sn.x, r1 = v1 * cc.x + v0 * sn.x;
        const float r2 = v2 * cc.y - v3 * sn.y, r3 = v3 * cc.y + v2 * sn.y;
        v0 = r0; v1 = r1; v2 = r2; v3 = r3;
      }
      y[e][0] = v0; y[e][1] = v1; y[e][2] = v2; y[e][3] = v3;
      ss = fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, fmaf(v3, v3, ss))));
    }
  }
  float r = 1.f;
  if (unit) r = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = (lane + 32 * e) * 4;
    if (c < dim) {
      Pack o;
#pragma unroll
      for (int i = 0; i < 4; ++i) o.v[i] = from_f32<T>(y[e][i] * r);
      *reinterpret_cast<Pack*>(row + c) = o;
    }
  }
}

// ------------------------------------------------------------------------------------------------ mean of normed outputs
// One CTA per token row: out = (1 / n) sum_j p_j / sqrt(mean(p_j^2) + eps) * w_j over up to four [T, W] tensors (each the
// 16-bit type T or fp32, its weight of the same type), fp32 out.
struct NormMeanArgs {
  const void* p[4];
  const void* w[4];
  int64_t ld[4];
  bool f32[4];
  int n;
};

// two parts whose rows fit the CTA's registers (W <= 256 x 4 x ITEMS): every input is read once
template <typename T, int ITEMS, int VEC>
__global__ void __launch_bounds__(256) norm_mean2_kernel(NormMeanArgs g, float* __restrict__ out, int W, float eps) {
  __shared__ float red[2 * 32];
  const int64_t t = blockIdx.x;
  float v[2][ITEMS][VEC];
  float ss[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int i = (it * 256 + threadIdx.x) * VEC;
      if (i < W) {
        load_vec<T, VEC>(g.p[j], g.f32[j], t * g.ld[j] + i, v[j][it]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss[j] = fmaf(v[j][it][e], v[j][it][e], ss[j]);
      }
    }
  block_sum<2>(ss, red);
  const float r0 = 0.5f / sqrtf(ss[0] / (float)W + eps), r1 = 0.5f / sqrtf(ss[1] / (float)W + eps);
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int i = (it * 256 + threadIdx.x) * VEC;
    if (i < W) {
      float w0[VEC], w1[VEC], acc[VEC];
      load_vec<T, VEC>(g.w[0], g.f32[0], i, w0);
      load_vec<T, VEC>(g.w[1], g.f32[1], i, w1);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = v[0][it][e] * r0 * w0[e] + v[1][it][e] * r1 * w1[e];
      store_vec<T, VEC>(out, true, t * W + i, acc);
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) norm_mean_kernel(NormMeanArgs g, float* __restrict__ out, int W, float eps) {
  __shared__ float red[4 * 32];
  const int64_t t = blockIdx.x;
  float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j < g.n) {
      for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
        float v[VEC];
        load_vec<T, VEC>(g.p[j], g.f32[j], t * g.ld[j] + i, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss[j] = fmaf(v[e], v[e], ss[j]);
      }
    }
  }
  block_sum<4>(ss, red);
  float r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) r[j] = 1.f / sqrtf(ss[j] / (float)W + eps);
  const float inv_n = 1.f / (float)g.n;
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < g.n) {
        float v[VEC], wv[VEC];
        load_vec<T, VEC>(g.p[j], g.f32[j], t * g.ld[j] + i, v);
        load_vec<T, VEC>(g.w[j], g.f32[j], i, wv);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += v[e] * r[j] * wv[e];
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] *= inv_n;
    store_vec<T, VEC>(out, true, t * W + i, acc);
  }
}

// ------------------------------------------------------------------------------------------------ sigmoid gate
template <typename T, int VEC>
__global__ void __launch_bounds__(256) sigmoid_gate_mul_kernel(T* __restrict__ o, const T* __restrict__ gate, int64_t ldg,
                                                               int64_t tokens, int C) {
  const int per = C / VEC;
  const int64_t total = tokens * per;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / per;
    const int c = (int)(idx % per) * VEC;
    float ov[VEC], gv[VEC];
    load_vec<T, VEC>(o, false, t * C + c, ov);
    load_vec<T, VEC>(gate, false, t * ldg + c, gv);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ov[e] *= sigmoid_f(gv[e]);
    store_vec<T, VEC>(o, false, t * C + c, ov);
  }
}

}  // namespace

// ================================================================================================ C launchers
extern "C" {

int cb_short_conv_silu(const void* x, int64_t ldx, const void* w, const void* bias, void* state, void* out, int64_t ldo,
                       const int* cu_q,
                       const int* ctx_len, const int* slots, int nseq, int max_q, int C, int taps, int apply_silu,
                       int update_state, int dtype, cudaStream_t st) {
  if (taps < 1 || taps > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (nseq == 0 || max_q == 0) return 0;
  dim3 grid((C + 127) / 128, (max_q + CONV_TOK_TILE - 1) / CONV_TOK_TILE, nseq);
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    const bool vec = taps <= CONV_VEC_TAPS && C % V == 0 && ldx % V == 0 && ldo % V == 0 && ((uintptr_t)x % 16) == 0 &&
                     ((uintptr_t)out % 16) == 0 && ((uintptr_t)state % 16) == 0;
    if (vec) {
      dim3 vgrid((C / V + 127) / 128, grid.y, grid.z);
      short_conv_silu_vec_kernel<T><<<vgrid, 128, 0, st>>>((const T*)x, ldx, (const T*)w, (const T*)bias, (const T*)state,
                                                          (T*)out, ldo, cu_q, ctx_len, slots, C, taps, apply_silu);
    } else {
      short_conv_silu_kernel<T><<<grid, 128, 0, st>>>((const T*)x, ldx, (const T*)w, (const T*)bias, (const T*)state,
                                                      (T*)out, ldo, cu_q, ctx_len, slots, C, taps, apply_silu);
    }
    if (update_state && taps > 1)
      short_conv_state_kernel<T><<<dim3((C + 127) / 128, nseq), 128, 0, st>>>((const T*)x, ldx, (T*)state, cu_q, ctx_len,
                                                                             slots, C, taps);
  });
  return CB_LAUNCH_CHECK();
}

// floats of workspace `cb_state_scan` needs for `tokens` tokens
int64_t cb_state_scan_workspace(int mode, int64_t tokens, int heads, int qk_heads, int dim, int vdim) {
  const int64_t DK = scan_dk(dim), VP = scan_vp(vdim);
  int64_t n = 2 * tokens * qk_heads * DK + tokens * heads * VP;
  if (mode == SCAN_DELTA) n += tokens * heads * DK + (tokens * heads + 3) / 4 * 4;
  if (mode == SCAN_GATED) n += tokens * heads * 4;
  return n;
}

int cb_state_scan(int mode, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                  const void* araw, int64_t lda, const void* braw, int64_t ldb, const float* head_decay,
                  const float* a_log, const float* dt_bias, float* state, float* out, float* work, int64_t tokens,
                  const int* cu_q, const int* ctx_len, const int* slots, int nseq, int heads, int qk_heads, int dim,
                  int vdim, int act_silu, int unit_qk, float unit_eps, float q_scale, float k_scale,
                  const float* rot_table, int rot_dims, const int* token_pos, int gate_kind, float gate_cap,
                  float* state_n, float* state_m, int dtype, cudaStream_t st) {
  if (nseq == 0 || tokens == 0) return 0;
  if (heads % qk_heads != 0 || rot_dims > dim || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
  if (mode == SCAN_GATED && ((gate_kind != GATE_STEP && gate_kind != GATE_EXP) || araw == nullptr || dt_bias == nullptr ||
                             (gate_kind == GATE_STEP && a_log == nullptr) ||
                             (gate_kind == GATE_EXP && (state_n == nullptr || state_m == nullptr))))
    return (int)cudaErrorInvalidValue;
  ScanParams p{q, k, v, ldq, ldk, ldv, araw, lda, braw, ldb, head_decay, a_log, dt_bias, state, out, cu_q, ctx_len, slots,
               heads, qk_heads, dim, vdim, act_silu, unit_qk, unit_eps, q_scale, k_scale, rot_table, rot_dims, token_pos,
               gate_kind, gate_cap, state_n, state_m};
  CB_DISPATCH_FLOAT(dtype, T, {
    if (mode == SCAN_GATED) return launch_scan<SCAN_GATED, T>(p, work, tokens, nseq, st);
    if (mode == SCAN_DELTA) return launch_scan<SCAN_DELTA, T>(p, work, tokens, nseq, st);
    return launch_scan<SCAN_DECAY, T>(p, work, tokens, nseq, st);
  });
  return CB_LAUNCH_CHECK();
}

int cb_gated_group_rmsnorm(const float* o, const void* w, int wn, const void* gate, int64_t ldg, void* out, int64_t tokens,
                           int C, int group, float eps, int gate_silu, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (group <= 0 || C % group != 0) return (int)cudaErrorInvalidValue;
  const int64_t units = tokens * (C / group);
  CB_DISPATCH_FLOAT(dtype, T, {
    const size_t al = 4 * sizeof(T);
    const bool wide = group >= 512 && group % 4 == 0 && ((uintptr_t)o & 15) == 0 && ((uintptr_t)out % al) == 0 &&
                      (gate == nullptr || (ldg % 4 == 0 && ((uintptr_t)gate % al) == 0));
    if (wide)
      gated_group_rmsnorm_wide_kernel<T><<<(unsigned)units, 256, 0, st>>>(o, (const T*)w, wn, (const T*)gate, ldg, (T*)out,
                                                                         C, group, eps, gate_silu);
    else
      gated_group_rmsnorm_kernel<T><<<(unsigned)((units + 7) / 8), 256, 0, st>>>(o, (const T*)w, wn, (const T*)gate, ldg,
                                                                                (T*)out, tokens, C, group, eps, gate_silu);
  });
  return CB_LAUNCH_CHECK();
}

int cb_rmsnorm_residual(float* x, const void* y, int64_t ldy, int y_f32, const void* w, void* h, int64_t tokens, int W,
                        int groups, float eps, float mult, float offset, const float* hist, int64_t hstride, int n,
                        const float* coef, float* mix_out, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (groups < 1 || W % groups != 0) return (int)cudaErrorInvalidValue;
  const int Wg = W / groups;
  const unsigned grid = (unsigned)(tokens * groups);
  CB_DISPATCH_FLOAT(dtype, T, {
    const size_t ysz = y_f32 ? sizeof(float) : sizeof(T);
    const bool vec = Wg % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)y % (4 * ysz)) == 0 &&
                     ((uintptr_t)w % (4 * sizeof(T))) == 0 && ((uintptr_t)h % (4 * sizeof(T))) == 0 && ((uintptr_t)x % 16) == 0 &&
                     ((uintptr_t)hist % 16) == 0 && ((uintptr_t)mix_out % 16) == 0 && hstride % 4 == 0 && W % 4 == 0;
    const int per = vec ? Wg / 4 : Wg;
    const int threads = per >= 256 ? 256 : (per + 31) / 32 * 32;
    if (y_f32) {
      if (vec)
        rmsnorm_residual_kernel<T, float, 4><<<grid, threads, 0, st>>>(x, (const float*)y, ldy, (const T*)w, (T*)h, W, groups,
                                                                      eps, mult, offset, hist, hstride, n, coef, mix_out);
      else
        rmsnorm_residual_kernel<T, float, 1><<<grid, threads, 0, st>>>(x, (const float*)y, ldy, (const T*)w, (T*)h, W, groups,
                                                                      eps, mult, offset, hist, hstride, n, coef, mix_out);
    } else if (vec) {
      rmsnorm_residual_kernel<T, T, 4><<<grid, threads, 0, st>>>(x, (const T*)y, ldy, (const T*)w, (T*)h, W, groups, eps,
                                                                mult, offset, hist, hstride, n, coef, mix_out);
    } else {
      rmsnorm_residual_kernel<T, T, 1><<<grid, threads, 0, st>>>(x, (const T*)y, ldy, (const T*)w, (T*)h, W, groups, eps,
                                                                mult, offset, hist, hstride, n, coef, mix_out);
    }
  });
  return CB_LAUNCH_CHECK();
}

int cb_rmsnorm_f32in(const float* x, int64_t ldx, const void* w, void* out, int64_t tokens, int W, int groups, float eps,
                     float offset, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (groups < 1 || W % groups != 0) return (int)cudaErrorInvalidValue;
  const int Wg = W / groups;
  const int threads = Wg >= 256 ? 256 : (Wg + 31) / 32 * 32;
  CB_DISPATCH_FLOAT(dtype, T, {
    rmsnorm_f32in_kernel<T><<<(unsigned)(tokens * groups), threads, 0, st>>>(x, ldx, (const T*)w, (T*)out, W, groups, eps,
                                                                            offset);
  });
  return CB_LAUNCH_CHECK();
}

int cb_depth_mix(const float* hist, int64_t stride, int n, const float* coef, float* out, void* h, int64_t total,
                 int dtype, cudaStream_t st) {
  if (total == 0) return 0;
  if (total % 4 != 0 || stride % 4 != 0 || ((uintptr_t)hist % 16) != 0 || ((uintptr_t)out % 16) != 0)
    return (int)cudaErrorInvalidValue;
  const int64_t total4 = total / 4;
  const unsigned grid = (unsigned)((total4 + 255) / 256 < 148 * 16 ? (total4 + 255) / 256 : 148 * 16);
  CB_DISPATCH_FLOAT(dtype, T, { depth_mix_kernel<T><<<grid, 256, 0, st>>>(hist, stride, n, coef, out, (T*)h, total4); });
  return CB_LAUNCH_CHECK();
}

int cb_poly_norm(const void* z, int64_t ldz, void* out, int64_t tokens, int F, const float* coef, float eps, int dtype,
                 cudaStream_t st) {
  if (tokens == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 16 / sizeof(T);
    const bool vec = F % V == 0 && ldz % V == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (vec) {
      const int nv = F / V;                       // vectors of a row: 2 per thread up to 256 threads, then 4, then 512 threads
      if (nv <= 512) {
        const int threads = (nv / 2 + 31) / 32 * 32;
        poly_norm_kernel<T, V, 2><<<(unsigned)tokens, threads < 32 ? 32 : threads, 0, st>>>((const T*)z, ldz, (T*)out, F,
                                                                                           coef, eps);
      } else {
        poly_norm_kernel<T, V, 4><<<(unsigned)tokens, nv <= 1024 ? 256 : 512, 0, st>>>((const T*)z, ldz, (T*)out, F, coef,
                                                                                      eps);
      }
    } else {
      poly_norm_kernel<T, 1, 4><<<(unsigned)tokens, 256, 0, st>>>((const T*)z, ldz, (T*)out, F, coef, eps);
    }
  });
  return CB_LAUNCH_CHECK();
}

int cb_head_rmsnorm(const void* x, int64_t ldx, void* out, int64_t ldo, int64_t tokens, int heads, int heads_a, int dim,
                    const void* wa, const void* wb, float eps, void* k_cache, void* v_cache, const int* block_tables,
                    const int* token_seq, const int* token_pos, int block_size, int max_blocks, int dtype,
                    cudaStream_t st) {
  if (tokens == 0 || heads == 0) return 0;
  const int64_t units = tokens * heads;
#define CB_HEAD_ARGS (const T*)x, ldx, (T*)out, ldo, tokens, heads, heads_a, dim, (const T*)wa, (const T*)wb, eps,     \
                     (T*)k_cache, (T*)v_cache, block_tables, token_seq, token_pos, block_size, max_blocks
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 8 / sizeof(T);              // 8-byte accesses: a warp covers a head of 128 16-bit channels at once
    const size_t al = V * sizeof(T);
    const bool vec = dim % V == 0 && ldx % V == 0 && ldo % V == 0 && ((uintptr_t)x % al) == 0 && ((uintptr_t)out % al) == 0 &&
                     ((uintptr_t)wa % al) == 0 && ((uintptr_t)wb % al) == 0 && ((uintptr_t)k_cache % al) == 0 &&
                     ((uintptr_t)v_cache % al) == 0;
    const unsigned grid = (unsigned)((units + 3) / 4);
    if (vec && dim <= 32 * V)
      head_rmsnorm_kernel<T, V, 1><<<grid, 128, 0, st>>>(CB_HEAD_ARGS);
    else if (vec)
      head_rmsnorm_kernel<T, V, 8><<<grid, 128, 0, st>>>(CB_HEAD_ARGS);
    else
      head_rmsnorm_kernel<T, 1, 4><<<grid, 128, 0, st>>>(CB_HEAD_ARGS);
  });
#undef CB_HEAD_ARGS
  return CB_LAUNCH_CHECK();
}

int cb_stream_add_norm(float* x, const void* a0, int64_t ld0, int dt0, const void* a1, int64_t ld1, int dt1, const void* a2,
                       int64_t ld2, int dt2, const void* a3, int64_t ld3, int dt3, const float* row, const void* w,
                       int w_dtype, void* h, int h_dtype, int64_t tokens, int W, int norm, float eps, float offset,
                       cudaStream_t st) {
  if (tokens == 0) return 0;
  if (norm < 0 || norm > 2 || (norm != 0 && h == nullptr)) return (int)cudaErrorInvalidValue;
  const void* ap[4] = {a0, a1, a2, a3};
  const int64_t ld[4] = {ld0, ld1, ld2, ld3};
  const int dts[4] = {dt0, dt1, dt2, dt3};
  // the one 16-bit type among addends, weight and output (fp32 operands may be mixed with it freely)
  int half_type = CB_F32;
  StreamArgs g;
  g.x = x;
  for (int j = 0; j < 4; ++j) {
    g.a[j] = ap[j];
    g.ld[j] = ld[j];
    g.a_f32[j] = dts[j] == CB_F32;
    if (ap[j] != nullptr && dts[j] != CB_F32) {
      if (half_type != CB_F32 && half_type != dts[j]) return (int)cudaErrorInvalidValue;
      half_type = dts[j];
    }
  }
  if (norm != 0) {
    if (w != nullptr && w_dtype != CB_F32) {
      if (half_type != CB_F32 && half_type != w_dtype) return (int)cudaErrorInvalidValue;
      half_type = w_dtype;
    }
    if (h_dtype != CB_F32) {
      if (half_type != CB_F32 && half_type != h_dtype) return (int)cudaErrorInvalidValue;
      half_type = h_dtype;
    }
  }
  g.row = row;
  g.w = norm != 0 ? w : nullptr;
  g.w_f32 = w_dtype == CB_F32;
  g.h = h;
  g.h_f32 = h_dtype == CB_F32;
  g.W = W;
  g.eps = eps;
  g.offset = offset;
  // four columns per access when every row start and width allows it
  bool vec = W % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)row & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
             ((uintptr_t)h & 15) == 0;
  for (int j = 0; j < 4; ++j) vec = vec && (ap[j] == nullptr || (ld[j] % 4 == 0 && ((uintptr_t)ap[j] & 15) == 0));
  CB_DISPATCH_FLOAT(half_type, T, {
    if (norm == 0) return launch_stream_add_norm<T, 0>(g, tokens, vec, st);
    if (norm == 1) return launch_stream_add_norm<T, 1>(g, tokens, vec, st);
    return launch_stream_add_norm<T, 2>(g, tokens, vec, st);
  });
  return CB_LAUNCH_CHECK();
}

int cb_rotary_half(const void* src, int64_t lds, void* dst, int64_t ldd, int64_t tokens, int heads, int src_hs, int src_off,
                   int dst_hs, int dst_off, int width, int dims, const float* table, const int* token_pos, int src_dtype,
                   int dst_dtype, cudaStream_t st) {
  if (tokens == 0 || heads == 0 || width == 0) return 0;
  if (dims > width || (dims & 1) || src_dtype != dst_dtype) return (int)cudaErrorInvalidValue;
  CB_DISPATCH_FLOAT(src_dtype, T, {
    constexpr int V = 16 / sizeof(T);
    const int half = dims / 2;
    const bool vec = half % V == 0 && (width - dims) % V == 0 && lds % V == 0 && ldd % V == 0 && src_hs % V == 0 &&
                     src_off % V == 0 && dst_hs % V == 0 && dst_off % V == 0 && ((uintptr_t)src & 15) == 0 &&
                     ((uintptr_t)dst & 15) == 0;
    const int64_t total = tokens * heads * ((half + (width - dims)) / (vec ? V : 1));
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    if (vec)
      rotary_half_kernel<T, V><<<grid, 256, 0, st>>>((const T*)src, lds, (T*)dst, ldd, tokens, heads, src_hs, src_off,
                                                     dst_hs, dst_off, width, dims, table, token_pos);
    else
      rotary_half_kernel<T, 1><<<grid, 256, 0, st>>>((const T*)src, lds, (T*)dst, ldd, tokens, heads, src_hs, src_off,
                                                     dst_hs, dst_off, width, dims, table, token_pos);
  });
  return CB_LAUNCH_CHECK();
}

int cb_latent_kv_write(const void* z, int64_t ldz, const void* w, int w_dtype, float eps, int rank, int rot,
                       const float* table, void* cache, const int* block_tables, const int* token_seq, const int* token_pos,
                       int64_t tokens, int block_size, int max_blocks, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (rot & 1) return (int)cudaErrorInvalidValue;
  const unsigned grid = (unsigned)((tokens + 7) / 8);
#define CB_LATENT_WRITE(T, TW, V)                                                                                     \
  latent_kv_write_kernel<T, TW, V><<<grid, 256, 0, st>>>((const T*)z, ldz, (const TW*)w, eps, rank, rot, table,        \
                                                         (T*)cache, block_tables, token_seq, token_pos, tokens,       \
                                                         block_size, max_blocks)
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 16 / sizeof(T);
    const bool vec = rank % V == 0 && (rank + rot) % V == 0 && ldz % V == 0 && ((uintptr_t)z & 15) == 0 &&
                     ((uintptr_t)cache & 15) == 0;
    if (w_dtype == CB_F32) {
      if (vec) CB_LATENT_WRITE(T, float, V); else CB_LATENT_WRITE(T, float, 1);
    } else if (w_dtype == dtype) {
      if (vec) CB_LATENT_WRITE(T, T, V); else CB_LATENT_WRITE(T, T, 1);
    } else {
      return (int)cudaErrorInvalidValue;
    }
  });
#undef CB_LATENT_WRITE
  return CB_LAUNCH_CHECK();
}

int cb_clamped_glu(const void* gu, void* out, int64_t rows, int I, float limit, float alpha, int dtype,
                   const int64_t* row_limit, cudaStream_t st) {
  if (rows == 0 || I == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 16 / sizeof(T);
    const bool vec = I % V == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0;
    const int64_t total = rows * (vec ? I / V : I);
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (vec) clamped_glu_kernel<T, V><<<grid, 256, 0, st>>>((const T*)gu, (T*)out, rows, I, limit, alpha, row_limit);
    else clamped_glu_kernel<T, 1><<<grid, 256, 0, st>>>((const T*)gu, (T*)out, rows, I, limit, alpha, row_limit);
  });
  return CB_LAUNCH_CHECK();
}

int cb_paged_kv_write_mix(const void* k, int64_t ldk, const void* v, int64_t ldv, const void* v_other, int64_t ldvo,
                          float lam, void* k_cache, void* v_cache, const int* block_tables, const int* token_seq,
                          const int* token_pos, int64_t tokens, int kw, int vw, int block_size, int max_blocks, int dtype,
                          cudaStream_t st) {
  if (tokens == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    paged_kv_write_mix_kernel<T><<<(unsigned)tokens, 128, 0, st>>>((const T*)k, ldk, (const T*)v, ldv, (const T*)v_other,
                                                                  ldvo, lam, (T*)k_cache, (T*)v_cache, block_tables,
                                                                  token_seq, token_pos, kw, vw, block_size, max_blocks);
  });
  return CB_LAUNCH_CHECK();
}

int cb_paged_bias_attention(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                            const int* token_seq, const int* token_pos, const float* bias_table, const int* bucket_start,
                            int nbuckets, void* out, int64_t tokens, int heads, int kv_heads, int dim, int vdim, int ldv,
                            int block_size, int max_blocks, float scale, int sink, int mask_block, const float* sink_vals,
                            const float* slopes, int window, int dtype, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (vdim > 32 * ATT_MAX_VREG || heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
  const int nwarps = 4;
  const size_t smem = (size_t)nwarps * dim * sizeof(float) + (size_t)nbuckets * sizeof(int);
  const int64_t units = tokens * heads;
  CB_DISPATCH_FLOAT(dtype, T, {
    paged_bias_attention_kernel<T><<<(unsigned)((units + nwarps - 1) / nwarps), nwarps * 32, smem, st>>>(
        (const T*)q, ldq, (const T*)k_cache, (const T*)v_cache, block_tables, token_seq, token_pos, bias_table,
        bucket_start, nbuckets, (T*)out, tokens, heads, kv_heads, dim, vdim, ldv, block_size, max_blocks, scale, sink,
        mask_block, sink_vals, slopes, window);
  });
  return CB_LAUNCH_CHECK();
}

// 16-bit dtypes, widths that are multiples of 8 and at most 256: the tensor-core kernel.  `chunk` > 0 (a multiple of 64)
// splits the keys over CTAs; part_o [tokens x heads x max_splits x vdim] and part_ml [.. x 2] are its fp32 workspace.
int cb_paged_bias_attention_mma(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                                const int* block_tables, const int* cu_q, const int* ctx_len, const int* token_pos,
                                const float* bias_table, const uint8_t* lut, int lut_n, int nbuckets, void* out,
                                int64_t tokens, int nseq, int max_q, int heads, int kv_heads, int dim, int vdim, int ldv,
                                int block_size, int max_blocks, float scale, int sink, int chunk, int max_splits,
                                float* part_o, float* part_ml, int mask_block, int wide_weights, const float* sink_vals,
                                const float* slopes, int window, int dtype, cudaStream_t st) {
  if (nseq == 0 || max_q == 0) return 0;
  if (heads % kv_heads != 0 || dim % 8 != 0 || vdim % 8 != 0 || dim > 256 || vdim > 256 || (ldq & 7) || ((uintptr_t)q & 15) ||
      (ldv & 7) || ldv < vdim ||
      chunk % MMA_BN != 0)
    return (int)cudaErrorInvalidValue;
  const int dmax = dim > vdim ? dim : vdim;
  const bool wide = max_q * (heads / kv_heads) > 64;      // 128 query rows per CTA (32 per warp) once a portion fills them
  const bool few = max_q * (heads / kv_heads) <= 16;      // decode steps: one m16 tile per sequence, warps split the keys
#define CB_ATT_MMA(T, D)                                                                                              \
  if (few)                                                                                                            \
    return launch_attention_mma<T, D, 1, true>(q, ldq, k_cache, v_cache, block_tables, cu_q, ctx_len, token_pos,       \
                                               bias_table, lut, lut_n, nbuckets, out, tokens, nseq, max_q, heads,      \
                                               kv_heads, dim, vdim, ldv, block_size, max_blocks, scale, sink, chunk,   \
                                               max_splits, part_o, part_ml, mask_block, wide_weights, sink_vals,       \
                                               slopes, window, st);                                                    \
  if (wide)                                                                                                           \
    return launch_attention_mma<T, D, 2>(q, ldq, k_cache, v_cache, block_tables, cu_q, ctx_len, token_pos, bias_table, \
                                         lut, lut_n, nbuckets, out, tokens, nseq, max_q, heads, kv_heads, dim, vdim,  \
                                         ldv, block_size, max_blocks, scale, sink, chunk, max_splits, part_o, part_ml, \
                                         mask_block, wide_weights, sink_vals, slopes, window, st);                    \
  return launch_attention_mma<T, D, 1>(q, ldq, k_cache, v_cache, block_tables, cu_q, ctx_len, token_pos, bias_table,  \
                                       lut, lut_n, nbuckets, out, tokens, nseq, max_q, heads, kv_heads, dim, vdim,   \
                                       ldv, block_size, max_blocks, scale, sink, chunk, max_splits, part_o, part_ml,  \
                                       mask_block, wide_weights, sink_vals, slopes, window, st)
  CB_DISPATCH_HALF(dtype, T, {
    if (dmax <= 32) { CB_ATT_MMA(T, 32); }
    else if (dmax <= 64) { CB_ATT_MMA(T, 64); }
    else if (dmax <= 128) { CB_ATT_MMA(T, 128); }
    else {                                               // 129..256 wide rows: one m16 tile per warp, one CTA per SM
      // (no key-splitting form here: at this width joining four 16 x 256 accumulators through shared memory costs more
      // than the three idle warps of a short decode CTA, measured 18.9 us against 14.1 us on 8 x 2048 keys)
      return launch_attention_mma<T, 256, 1>(q, ldq, k_cache, v_cache, block_tables, cu_q, ctx_len, token_pos, bias_table,
                                             lut, lut_n, nbuckets, out, tokens, nseq, max_q, heads, kv_heads, dim, vdim,
                                             ldv, block_size, max_blocks, scale, sink, chunk, max_splits, part_o, part_ml,
                                             mask_block, wide_weights, sink_vals, slopes, window, st);
    }
  });
#undef CB_ATT_MMA
  return CB_LAUNCH_CHECK();
}

int cb_lru_scan(const void* u, int64_t ldu, const float* gates, const float* gbias, const float* lam, const void* branch,
                int64_t ldb, float* state, void* out, int64_t tokens, const int* cu_q, const int* ctx_len, const int* slots,
                int nseq, int C, int nb, float cmul, int dtype, cudaStream_t st) {
  if (nseq == 0 || tokens == 0) return 0;
  if (nb <= 0 || C % nb != 0) return (int)cudaErrorInvalidValue;
  dim3 grid((C + 127) / 128, nseq);
  CB_DISPATCH_FLOAT(dtype, T, {
    lru_scan_kernel<T><<<grid, 128, 0, st>>>((const T*)u, ldu, gates, gbias, lam, (const T*)branch, ldb, state, (T*)out,
                                             tokens, cu_q, ctx_len, slots, C, nb, cmul);
  });
  return CB_LAUNCH_CHECK();
}

int cb_rotary_unit_norm(void* x, int64_t ldx, int64_t tokens, int heads, int dim, int rot_dims, int interleaved,
                        const float* table, const int* token_pos, int unit, float eps, int dtype, cudaStream_t st) {
  if (tokens == 0 || heads == 0) return 0;
  if (dim > 32 * ROT_MAX_REG || rot_dims > dim || (rot_dims & 1) || (rot_dims > 0 && table == nullptr))
    return (int)cudaErrorInvalidValue;
  const int64_t items = tokens * heads;
  CB_DISPATCH_FLOAT(dtype, T, {
    const size_t al = 4 * sizeof(T);
    const bool vec = (interleaved || rot_dims == 0) && dim % 4 == 0 && rot_dims % 4 == 0 && ldx % 4 == 0 &&
                     ((uintptr_t)x % al) == 0 && ((uintptr_t)table & 7) == 0;
    if (vec)
      rotary_pairs_unit_norm_kernel<T><<<(unsigned)((items + 3) / 4), 128, 0, st>>>((T*)x, ldx, tokens, heads, dim, rot_dims,
                                                                                   table, token_pos, unit, eps);
    else
      rotary_unit_norm_kernel<T><<<(unsigned)((items + 3) / 4), 128, (size_t)4 * dim * sizeof(float), st>>>(
          (T*)x, ldx, tokens, heads, dim, rot_dims, interleaved, table, token_pos, unit, eps);
  });
  return CB_LAUNCH_CHECK();
}

int cb_norm_mean(const void* p0, int64_t ld0, const void* w0, int dt0, const void* p1, int64_t ld1, const void* w1, int dt1,
                 const void* p2, int64_t ld2, const void* w2, int dt2, const void* p3, int64_t ld3, const void* w3, int dt3,
                 int n, float* out, int64_t tokens, int W, float eps, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (n < 1 || n > 4) return (int)cudaErrorInvalidValue;
  NormMeanArgs g;
  const void* ps[4] = {p0, p1, p2, p3};
  const void* ws[4] = {w0, w1, w2, w3};
  const int64_t lds[4] = {ld0, ld1, ld2, ld3};
  const int dts[4] = {dt0, dt1, dt2, dt3};
  int half_type = CB_F32;
  bool vec = W % 4 == 0 && ((uintptr_t)out & 15) == 0;
  for (int j = 0; j < 4; ++j) {
    g.p[j] = ps[j]; g.w[j] = ws[j]; g.ld[j] = lds[j]; g.f32[j] = dts[j] == CB_F32;
    if (j >= n) continue;
    if (ps[j] == nullptr || ws[j] == nullptr) return (int)cudaErrorInvalidValue;
    if (dts[j] != CB_F32) {
      if (half_type != CB_F32 && half_type != dts[j]) return (int)cudaErrorInvalidValue;
      half_type = dts[j];
    }
    const size_t es = dts[j] == CB_F32 ? 4 : 2;
    vec = vec && lds[j] % 4 == 0 && ((uintptr_t)ps[j] % (4 * es)) == 0 && ((uintptr_t)ws[j] % (4 * es)) == 0;
  }
  g.n = n;
  if (half_type == CB_F32) half_type = CB_BF16;      // no 16-bit operand: the type only names the unused branch
  CB_DISPATCH_HALF(half_type, T, {
    // 16-byte reads of two 16-bit parts where widths and addresses allow, else 8-byte ones
    bool vec8 = vec && n == 2 && W % 8 == 0 && ((uintptr_t)out & 31) == 0;
    for (int j = 0; j < 2 && vec8; ++j)
      vec8 = dts[j] != CB_F32 && lds[j] % 8 == 0 && ((uintptr_t)ps[j] & 15) == 0 && ((uintptr_t)ws[j] & 15) == 0;
    if (vec8 && W <= 2048) norm_mean2_kernel<T, 1, 8><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec8 && W <= 4096) norm_mean2_kernel<T, 2, 8><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec8 && W <= 8192) norm_mean2_kernel<T, 4, 8><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec && n == 2 && W <= 1024) norm_mean2_kernel<T, 1, 4><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec && n == 2 && W <= 2048) norm_mean2_kernel<T, 2, 4><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec && n == 2 && W <= 4096) norm_mean2_kernel<T, 4, 4><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec && n == 2 && W <= 8192) norm_mean2_kernel<T, 8, 4><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else if (vec) norm_mean_kernel<T, 4><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
    else norm_mean_kernel<T, 1><<<(unsigned)tokens, 256, 0, st>>>(g, out, W, eps);
  });
  return CB_LAUNCH_CHECK();
}

int cb_sigmoid_gate_mul(void* o, const void* gate, int64_t ldg, int64_t tokens, int C, int dtype, cudaStream_t st) {
  if (tokens == 0 || C == 0) return 0;
  CB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 16 / sizeof(T);
    const bool vec = C % V == 0 && ldg % V == 0 && ((uintptr_t)o & 15) == 0 && ((uintptr_t)gate & 15) == 0;
    const int64_t total = tokens * (vec ? C / V : C);
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (vec) sigmoid_gate_mul_kernel<T, V><<<grid, 256, 0, st>>>((T*)o, (const T*)gate, ldg, tokens, C);
    else sigmoid_gate_mul_kernel<T, 1><<<grid, 256, 0, st>>>((T*)o, (const T*)gate, ldg, tokens, C);
  });
  return CB_LAUNCH_CHECK();
}

}  // extern "C"
