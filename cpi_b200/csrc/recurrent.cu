// Recurrent mixers: a short causal convolution with carried inputs, a linear recurrence over a matrix state
// per head, and the gated norm that follows it.
//
//   causal_conv        out[t, c] = act(bias[c] + sum_j w[c, j] * in[t - (taps - 1) + j, c]); inputs before a
//                      step's first token come from the sequence's carried inputs (the last taps - 1 of the
//                      steps before, zeros at the start of the sequence).
//   conv_carry         after the convolution: the carried inputs become the last taps - 1 inputs seen so far.
//   linear_scan        per sequence and head, a state S [N rows, Dv columns] in float32 that lives in a slot:
//                        S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t (+ skip * v_t)
//                      in two flavours: a decay per row, a_t = sigmoid(z_t + bias)^(1 / tau) (gated linear
//                      attention; q scaled by a constant), or one decay per head with a step size,
//                      dt = softplus(raw_t + dt_bias), a_t = exp(-exp(A_log) dt), v_t' = dt v_t (the selective
//                      state-space form, where k is called B, q is called C and heads share B and C in groups).
//                      Decays, step sizes and the state are float32 whatever the activations are.
//                      A row decay may also be a_t = exp(-exp(A_log[head]) * softplus(z_t + bias)).  With `beta`
//                      the update is the delta rule: after the decay, u_t = beta_t (v_t - S^T k_t), S += k_t u_t^T,
//                      o_t = S^T q_t (the read-out sees the token's own write).
//   rglru_scan         a gated linear recurrent unit with one state element per channel (see its own comment);
//   block_major_rows   the equal parts of float32 rows laid out part by part, as the rows of a grouped product.
//   head_unit          rows of heads made unit vectors in place: x / sqrt(sum(x^2) + eps) per head.
//   gated_norm         out = norm_g(y * act(g)) * w  or  norm_g(y) * w * act(g): an RMS norm over equal parts
//                      of a row (each part by its own mean square), gate before or after; act is silu or sigmoid.
//
// A sequence's tokens are visited in order by one block per (sequence, head, slice of columns) with the same
// arithmetic whether they come in one step or one at a time, so results do not depend on how a prompt is cut.
#include "common.cuh"

namespace cpi {

constexpr int CONV_MAX_TAPS = 8;

struct ConvParams {
  const float* in; long in_stride;       // [T, C] (a column slice of a wider row)
  const void* w; const void* bias; int w_dtype;      // [C, taps], [C] or null
  float* carry;                          // [slots, taps - 1, C] float32
  const int* token_seq; const int* token_pos; const int* seq_slot; const int* seq_start;
  const int* seq_tok0; const int* seq_new;
  float* out; long out_stride;           // [T, C] float32
  int channels, taps, silu;
  const void* in_bias;                   // [C] or null (w's dtype): added to every input of the step before it is used or carried
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__global__ void __launch_bounds__(256) causal_conv_kernel(ConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.channels) return;
  const int s = p.token_seq[t];
  const int local = p.token_pos[t] - p.seq_start[s];          // tokens of this sequence before t in this step
  const float* carry = p.carry + (size_t)p.seq_slot[s] * (p.taps - 1) * p.channels;
  float acc = p.bias ? load_any(p.bias, p.w_dtype, c) : 0.f;
  const float ib = p.in_bias ? load_any(p.in_bias, p.w_dtype, c) : 0.f;
  for (int j = 0; j < p.taps; ++j) {
    const int back = p.taps - 1 - j;                          // how many tokens before t
    float x;
    if (back <= local) x = p.in[(size_t)(t - back) * p.in_stride + c] + ib;
    else x = carry[(size_t)(p.taps - 1 - (back - local)) * p.channels + c];
    acc = fmaf(load_any(p.w, p.w_dtype, (size_t)c * p.taps + j), x, acc);
  }
  p.out[(size_t)t * p.out_stride + c] = p.silu ? silu_f(acc) : acc;
}

__global__ void __launch_bounds__(256) conv_carry_kernel(ConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.channels) return;
  const int n = p.seq_new[s], tok0 = p.seq_tok0[s], keep = p.taps - 1;
  float* carry = p.carry + (size_t)p.seq_slot[s] * keep * p.channels;
  float v[CONV_MAX_TAPS];
  const float ib = p.in_bias ? load_any(p.in_bias, p.w_dtype, c) : 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    if (j < keep) {
      const int idx = n - keep + j;                           // index among this step's tokens; negative: an older input
      v[j] = idx >= 0 ? p.in[(size_t)(tok0 + idx) * p.in_stride + c] + ib : carry[(size_t)(j + n) * p.channels + c];
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
    if (j < keep) carry[(size_t)j * p.channels + c] = v[j];
}

// ---- the recurrence ---------------------------------------------------------------------------------------
struct ScanParams {
  const float* k; long k_stride;         // [T, groups * N]
  const float* q; long q_stride;         // [T, groups * N]
  const float* v; long v_stride;         // [T, H * Dv]
  const float* z; long z_stride;         // row decays before the sigmoid [T, H * N]      (row flavour)
  const void* z_bias; float inv_tau;     // [H * N] or null
  const float* dt; long dt_stride;       // raw step sizes [T, H]                         (head flavour)
  const void* dt_bias; const void* a_log; const void* skip;      // [H] each; skip may be null
  int small_dtype;                       // dtype of z_bias, dt_bias, a_log, skip
  float q_scale;
  float* state;                          // [slots, H, N, Dv]
  float* out; long out_stride;           // [T, H * Dv]
  const int* seq_slot; const int* seq_tok0; const int* seq_new;
  int n_heads, heads_per_group, n_rows, n_cols;      // H, H / groups, N, Dv
  int chunk;                             // tokens staged in shared memory at a time
  int vec16;                             // the rows of k, q and z start on 16-byte boundaries and N is a multiple of 4
  int decay_ready;                       // z already holds the decays a (row_decay ran over it)
  int decay_kind;                        // row flavour: 0 a = sigmoid(z + b)^(1/tau), 1 a = exp(-exp(a_log[head]) softplus(z + b))
  const float* beta; long beta_stride;   // [T, H] before the sigmoid, or null; with it the update is the delta rule
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
// a = sigmoid(z + b)^(1 / tau); one function for the kernel that prepares a prompt's decays and for the recurrence
// that computes a decoded token's own, so that both give the same bits
// (kind 1: a = exp(-rate * softplus(z + b)), rate = exp(A_log) of the row's head)
__device__ __forceinline__ float row_decay_f(float z, float b, float inv_tau, int kind = 0, float rate = 0.f) {
  if (kind == 1) return expf(-rate * softplus_f(z + b));
  return expf(log_sigmoid_f(z + b) * inv_tau);
}

struct RowDecayParams {
  float* z; long z_stride; const void* bias; int bias_dtype; float inv_tau; int n;
  int kind; const void* a_log; int rows_per_head;       // kind 1: element i belongs to head i / rows_per_head
};

// z[t, i] <- sigmoid(z[t, i] + bias[i])^(1 / tau), in place: the decays of a step of many tokens, once per element
// instead of once per block of columns inside the recurrence
__global__ void __launch_bounds__(256) row_decay_kernel(RowDecayParams p) {
  // (no early launch of the kernel behind it: that is the recurrence of a prompt, whose few blocks would be placed
  // on whichever multiprocessors this kernel's blocks leave first, several to one, instead of one each; measured:
  // 1.09 instead of 0.60 ms for the delta rule at 2,048 tokens)
  pdl_wait();
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= p.n) return;
  float* z = p.z + (size_t)blockIdx.x * p.z_stride + i;
  const float rate = p.kind == 1 ? expf(load_any(p.a_log, p.bias_dtype, i / p.rows_per_head)) : 0.f;
  *z = row_decay_f(*z, p.bias ? load_any(p.bias, p.bias_dtype, i) : 0.f, p.inv_tau, p.kind, rate);
}

__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst_smem))), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst_smem))), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Threads of a warp: lane = kk * PVW + pp with KS lanes (kk) sharing a column and PVW = 32 / KS columns (pp) per
// warp.  Lane kk owns the state rows kk * NPT .. kk * NPT + NPT - 1 of its column in registers.  Tokens come
// through shared memory a chunk at a time, in two buffers: while one chunk is computed the next one's rows (k, q,
// the decays before their transform, the block's columns of v, the raw step sizes) are on their way as
// asynchronous copies, 16 bytes each where the rows allow it.  Once a chunk has landed, one pass turns what was
// copied into what the recurrence needs (a = sigmoid(z + b)^(1/tau) unless the caller prepared it, or the step
// size and the head's decay); q's constant scale multiplies the output sum.  Per token the rows' k, q and a lie as each lane group's NPT values followed by four words of padding,
// so that the 16-byte reads of different kk fall into different banks.
template <int NPT, int KS, bool ROW_DECAY, int CPT, bool DELTA>
__global__ void __launch_bounds__(256) linear_scan_kernel(ScanParams p) {
  // A decode step (one token staged at a time) lets the kernel behind it start at once.  A prompt does not: its few
  // blocks run for hundreds of microseconds, one to a multiprocessor, on a chain of dependent instructions, and
  // thousands of blocks of the next kernel waiting beside them were measured to slow that chain by half.
  if (p.chunk == 1) pdl_launch_dependents();
  extern __shared__ __align__(16) float smem[];
  constexpr int PVW = 32 / KS, ROWP = KS * (NPT + 4), NVEC = ROW_DECAY ? 3 : 2;
  const int nwarps = blockDim.x >> 5, pvb = nwarps * PVW * CPT;
  const int s = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, kk = lane / PVW, pp = lane % PVW;
  const int lcol = (warp * PVW + pp) * CPT;                  // this thread's first column within the block's slice
  const int col0 = blockIdx.z * pvb, col = col0 + lcol;
  const int N = p.n_rows, Dv = p.n_cols, H = p.n_heads, g = h / p.heads_per_group;
  const int chunk = p.chunk;
  const int per_buf = (chunk * (NVEC * ROWP + pvb + 2) + 3) & ~3;
  float* bias_s = smem + 2 * per_buf;                        // [KS * NPT] the decays' bias (row flavour)
  auto k_of = [&](float* b) { return b; };
  auto q_of = [&](float* b) { return b + (size_t)chunk * ROWP; };
  auto d_of = [&](float* b) { return b + (size_t)2 * chunk * ROWP; };
  auto v_of = [&](float* b) { return b + (size_t)NVEC * chunk * ROWP; };
  auto dt_of = [&](float* b) { return b + (size_t)NVEC * chunk * ROWP + (size_t)chunk * pvb; };
  auto a_of = [&](float* b) { return dt_of(b) + chunk; };

  // what no kernel writes comes before the wait: the head's constants, the bias; the buffers start as zeros
  // (rows past the state's size and columns past the head's are never copied into and stay zero)
  float head_a = 0.f, head_dtb = 0.f, head_skip = 0.f, head_rate = 0.f;
  if (ROW_DECAY && p.decay_kind == 1) head_rate = expf(load_any(p.a_log, p.small_dtype, h));
  if (!ROW_DECAY) {
    head_a = -expf(load_any(p.a_log, p.small_dtype, h));
    head_dtb = p.dt_bias ? load_any(p.dt_bias, p.small_dtype, h) : 0.f;
  }
  if (p.skip) head_skip = load_any(p.skip, p.small_dtype, h);
  for (int i = tid; i < 2 * per_buf; i += blockDim.x) smem[i] = 0.f;
  if (ROW_DECAY)
    for (int n = tid; n < KS * NPT; n += blockDim.x)
      bias_s[n] = (n < N && p.z_bias) ? load_any(p.z_bias, p.small_dtype, (size_t)h * N + n) : 0.f;
  pdl_wait();
  const int n_tok = p.seq_new[s], tok0 = p.seq_tok0[s];
  float* st = p.state + (((size_t)p.seq_slot[s] * H + h) * N) * Dv + col;
  // rows kk * NPT .., columns col .. col + CPT - 1; two neighbouring rows of a column make one pair, so that the
  // recurrence runs on the packed float32 instructions (each half rounds as the single instruction does)
  float2 S[NPT / 2][CPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = kk * NPT + i;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const float s0 = (col + c < Dv && n < N) ? st[(size_t)n * Dv + c] : 0.f;
      if (i & 1) S[i / 2][c].y = s0; else S[i / 2][c].x = s0;
    }
  }
  __syncthreads();                                           // the zeros are in place before the first copies land

  auto issue = [&](int c0, float* b) {
    const int nc = min(chunk, n_tok - c0);
    float *ks = k_of(b), *qs = q_of(b), *ds = d_of(b);
    if (p.vec16) {
      constexpr int G4 = KS * NPT / 4;
      for (int e = tid; e < nc * G4; e += blockDim.x) {
        const int j = e / G4, n = (e % G4) * 4;
        if (n >= N) continue;
        const int at = j * ROWP + (n / NPT) * (NPT + 4) + n % NPT;
        const size_t t = (size_t)(tok0 + c0 + j);
        cp_async16(ks + at, p.k + t * p.k_stride + (size_t)g * N + n);
        cp_async16(qs + at, p.q + t * p.q_stride + (size_t)g * N + n);
        if (ROW_DECAY) cp_async16(ds + at, p.z + t * p.z_stride + (size_t)h * N + n);
      }
    } else {
      for (int e = tid; e < nc * KS * NPT; e += blockDim.x) {
        const int j = e / (KS * NPT), n = e % (KS * NPT);
        if (n >= N) continue;
        const int at = j * ROWP + (n / NPT) * (NPT + 4) + n % NPT;
        const size_t t = (size_t)(tok0 + c0 + j);
        cp_async4(ks + at, p.k + t * p.k_stride + (size_t)g * N + n);
        cp_async4(qs + at, p.q + t * p.q_stride + (size_t)g * N + n);
        if (ROW_DECAY) cp_async4(ds + at, p.z + t * p.z_stride + (size_t)h * N + n);
      }
    }
    float* vs = v_of(b);
    for (int e = tid; e < nc * pvb; e += blockDim.x) {
      const int j = e / pvb, c = col0 + e % pvb;
      if (c < Dv) cp_async4(vs + e, p.v + (size_t)(tok0 + c0 + j) * p.v_stride + (size_t)h * Dv + c);
    }
    if (!ROW_DECAY) {
      float* dts = dt_of(b);
      for (int j = tid; j < nc; j += blockDim.x) cp_async4(dts + j, p.dt + (size_t)(tok0 + c0 + j) * p.dt_stride + h);
    }
    if (DELTA) {                                             // the place of the step sizes holds the write strengths
      float* bs = dt_of(b);
      for (int j = tid; j < nc; j += blockDim.x) cp_async4(bs + j, p.beta + (size_t)(tok0 + c0 + j) * p.beta_stride + h);
    }
  };

  if (n_tok > 0) issue(0, smem);
  cp_async_commit();
  int which = 0;
  for (int c0 = 0; c0 < n_tok; c0 += chunk, which ^= 1) {
    float* b = smem + which * per_buf;
    const int nc = min(chunk, n_tok - c0);
    if (c0 + chunk < n_tok) issue(c0 + chunk, smem + (which ^ 1) * per_buf);
    cp_async_commit();
    cp_async_wait<1>();                                      // this chunk's copies (the group before the newest) are done
    __syncthreads();
    // what was copied becomes what the recurrence needs
    float *ks = k_of(b), *qs = q_of(b), *ds = d_of(b), *vs = v_of(b), *dts = dt_of(b), *as = a_of(b);
    const bool transform = ROW_DECAY ? !p.decay_ready : true;
    if (ROW_DECAY && transform) {
      for (int e = tid; e < nc * KS * NPT; e += blockDim.x) {
        const int j = e / (KS * NPT), n = e % (KS * NPT);
        if (n >= N) continue;
        const int at = j * ROWP + (n / NPT) * (NPT + 4) + n % NPT;
        ds[at] = row_decay_f(ds[at], bias_s[n], p.inv_tau, p.decay_kind, head_rate);
      }
    }
    if (DELTA)
      for (int j = tid; j < nc; j += blockDim.x) dts[j] = 1.0f / (1.0f + expf(-dts[j]));
    if (!ROW_DECAY) {
      for (int j = tid; j < nc; j += blockDim.x) {
        const float dt = softplus_f(dts[j] + head_dtb);
        dts[j] = dt;
        as[j] = expf(head_a * dt);
      }
    }
    if (transform || DELTA) __syncthreads();
#pragma unroll 2
    for (int j = 0; j < nc; ++j) {
      const float4* k4 = reinterpret_cast<const float4*>(ks + j * ROWP + kk * (NPT + 4));
      const float4* q4 = reinterpret_cast<const float4*>(qs + j * ROWP + kk * (NPT + 4));
      const float4* d4 = reinterpret_cast<const float4*>(ds + j * ROWP + kk * (NPT + 4));
      float v_raw[CPT], o[CPT];
      float2 vv[CPT], o2[CPT];
      float a = 0.f, dtj = 1.f;
      if (!ROW_DECAY) { dtj = dts[j]; a = as[j]; }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        v_raw[c] = vs[j * pvb + lcol + c];
        vv[c] = make_float2(v_raw[c] * dtj, v_raw[c] * dtj);
        o2[c] = make_float2(0.f, 0.f);
      }
      if constexpr (DELTA) {
        // The delta rule.  One pass over the thread's rows decays them and takes, for every column, what the decayed
        // state answers to this token's key (d) and to its query (e), and once per thread its share of k . q.  After
        // the sums over the lanes that share a column, u = beta (v - d) is what the token writes, and its output is
        // S'^T q = e + (k . q) u: the read-out of the updated state without a second sum over it.  The second pass
        // only adds k u^T to the rows.
        float2 d2[CPT], kq2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < CPT; ++c) d2[c] = make_float2(0.f, 0.f);
#pragma unroll
        for (int i4 = 0; i4 < NPT / 4; ++i4) {
          const float4 kq = k4[i4], qq = q4[i4];
          float4 dd = make_float4(a, a, a, a);
          if (ROW_DECAY) dd = d4[i4];
          const float2 kr[2] = {make_float2(kq.x, kq.y), make_float2(kq.z, kq.w)};
          const float2 qr[2] = {make_float2(qq.x, qq.y), make_float2(qq.z, qq.w)};
          const float2 dr[2] = {make_float2(dd.x, dd.y), make_float2(dd.z, dd.w)};
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            kq2 = __ffma2_rn(kr[r], qr[r], kq2);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
              S[2 * i4 + r][c] = __fmul2_rn(dr[r], S[2 * i4 + r][c]);
              d2[c] = __ffma2_rn(S[2 * i4 + r][c], kr[r], d2[c]);
              o2[c] = __ffma2_rn(S[2 * i4 + r][c], qr[r], o2[c]);
            }
          }
        }
        const float beta = dts[j];
        float kqs = kq2.x + kq2.y;
#pragma unroll
        for (int off = PVW; off < 32; off <<= 1) kqs += __shfl_xor_sync(0xffffffffu, kqs, off);
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          float d = d2[c].x + d2[c].y, e = o2[c].x + o2[c].y;
#pragma unroll
          for (int off = PVW; off < 32; off <<= 1) {
            d += __shfl_xor_sync(0xffffffffu, d, off);
            e += __shfl_xor_sync(0xffffffffu, e, off);
          }
          const float u = beta * (v_raw[c] - d);
          vv[c] = make_float2(u, u);
          o[c] = fmaf(kqs, u, e);
          if (kk == 0 && col + c < Dv)
            p.out[(size_t)(tok0 + c0 + j) * p.out_stride + (size_t)h * Dv + col + c] = fmaf(head_skip, v_raw[c], o[c] * p.q_scale);
        }
#pragma unroll
        for (int i4 = 0; i4 < NPT / 4; ++i4) {
          const float4 kq = k4[i4];
          const float2 kr[2] = {make_float2(kq.x, kq.y), make_float2(kq.z, kq.w)};
#pragma unroll
          for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) S[2 * i4 + r][c] = __ffma2_rn(kr[r], vv[c], S[2 * i4 + r][c]);
          }
        }
      } else {
      // a thread's rows times its columns: k, q and the decay of a row are read once for all its columns
#pragma unroll
      for (int i4 = 0; i4 < NPT / 4; ++i4) {
        const float4 kq = k4[i4], qq = q4[i4];
        float4 dd = make_float4(a, a, a, a);
        if (ROW_DECAY) dd = d4[i4];
        const float2 kr[2] = {make_float2(kq.x, kq.y), make_float2(kq.z, kq.w)};
        const float2 qr[2] = {make_float2(qq.x, qq.y), make_float2(qq.z, qq.w)};
        const float2 dr[2] = {make_float2(dd.x, dd.y), make_float2(dd.z, dd.w)};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            S[2 * i4 + r][c] = __ffma2_rn(kr[r], vv[c], __fmul2_rn(dr[r], S[2 * i4 + r][c]));
            o2[c] = __ffma2_rn(S[2 * i4 + r][c], qr[r], o2[c]);
          }
        }
      }
      }
      if constexpr (!DELTA) {                                // (the delta rule has stored its outputs above)
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        o[c] = o2[c].x + o2[c].y;
#pragma unroll
        for (int off = PVW; off < 32; off <<= 1) o[c] += __shfl_xor_sync(0xffffffffu, o[c], off);
        if (kk == 0 && col + c < Dv)
          p.out[(size_t)(tok0 + c0 + j) * p.out_stride + (size_t)h * Dv + col + c] = fmaf(head_skip, v_raw[c], o[c] * p.q_scale);
      }
      }
    }
    __syncthreads();                                         // the buffer may be copied into again
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = kk * NPT + i;
#pragma unroll
    for (int c = 0; c < CPT; ++c)
      if (col + c < Dv && n < N) st[(size_t)n * Dv + c] = (i & 1) ? S[i / 2][c].y : S[i / 2][c].x;
  }
}

// ---- gated norm -------------------------------------------------------------------------------------------
struct GatedNormParams {
  const float* y; long y_stride;         // [T, width]
  const float* gate; long gate_stride;   // [T, width] or null
  const void* w; int w_dtype; int w_len; // weight index = i % w_len (a weight shared by all parts, or one per element)
  void* out; long out_stride;
  int width, parts, gate_first; float eps;
  int gate_act;                          // 0 silu, 1 sigmoid
};

__device__ __forceinline__ float gate_f(float z, int act) { return act == 1 ? 1.0f / (1.0f + expf(-z)) : silu_f(z); }

template <typename TO>
__global__ void __launch_bounds__(128) gated_norm_kernel(GatedNormParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = blockIdx.y, n = p.width / p.parts;
  const float* y = p.y + (size_t)t * p.y_stride + (size_t)part * n;
  const float* g = p.gate ? p.gate + (size_t)t * p.gate_stride + (size_t)part * n : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = y[i];
    if (g && p.gate_first) v *= gate_f(g[i], p.gate_act);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + p.eps);
  TO* o = reinterpret_cast<TO*>(p.out) + (size_t)t * p.out_stride + (size_t)part * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = y[i];
    if (g && p.gate_first) v *= gate_f(g[i], p.gate_act);
    v *= inv;
    if (p.w) v *= load_any(p.w, p.w_dtype, (size_t)(part * n + i) % p.w_len);
    if (g && !p.gate_first) v *= gate_f(g[i], p.gate_act);
    o[i] = from_f32<TO>(v);
  }
}

// x[t, head, :] <- x / sqrt(sum(x^2) + eps) in place, float32 rows of `heads` heads of `dim` elements; a warp per head
__global__ void __launch_bounds__(128) head_unit_kernel(float* x, long stride, int heads, int dim, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= heads) return;
  float* r = x + (size_t)blockIdx.x * stride + (size_t)head * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(r[i], r[i], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) + eps);
  for (int i = lane; i < dim; i += 32) r[i] *= inv;
}

template <int NPT, int KS, bool ROW, int CPT = 1>
static int launch_scan(const ScanParams& p0, int n_seqs, int max_new, int max_warps, cudaStream_t stream) {
  ScanParams p = p0;
  constexpr int PVW = 32 / KS, ROWP = KS * (NPT + 4);
  int nwarps = (p.n_cols + PVW * CPT - 1) / (PVW * CPT);
  if (nwarps > max_warps) nwarps = max_warps;
  const int pvb = nwarps * PVW * CPT;
  const int per_token = (ROW ? 3 : 2) * ROWP + pvb + 2;
  int chunk = (36 * 1024 / 4) / per_token;                   // two buffers of this many tokens: three blocks share an SM
  if (chunk > 16) chunk = 16;
  if (chunk > max_new) chunk = max_new;                      // a decode step stages one token: small blocks, all resident
  if (chunk < 1) chunk = 1;
  p.chunk = chunk;
  const int per_buf = (chunk * per_token + 3) & ~3;
  const size_t smem = ((size_t)2 * per_buf + KS * NPT) * sizeof(float);
  auto aligned = [](const float* q, long stride) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0 && stride % 4 == 0; };
  p.vec16 = p.n_rows % 4 == 0 && aligned(p.k, p.k_stride) && aligned(p.q, p.q_stride) && (!ROW || aligned(p.z, p.z_stride));
  auto kern = ROW && p.beta ? linear_scan_kernel<NPT, KS, ROW, CPT, ROW> : linear_scan_kernel<NPT, KS, ROW, CPT, false>;
  static bool attr_set[2] = {false, false};                  // per instantiation
  if (smem > 48 * 1024 && !attr_set[p.beta != nullptr]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
      set_error("linear_scan: %zu bytes of shared memory were refused", smem);
      return 1;
    }
    attr_set[p.beta != nullptr] = true;
  }
  dim3 grid(n_seqs, p.n_heads, (p.n_cols + pvb - 1) / pvb);
  cpi::launch_pdl(kern, grid, dim3(32 * nwarps), smem, stream, p);
  return check_launch("linear_scan");
}

// Two shapes of block.  Narrow: four lanes share a column, each with a quarter of the rows in registers, two warps
// (16 columns) per block: the most columns per byte of staging, for steps with many sequences.  Wide: sixteen
// lanes share a column, eight warps (16 columns) per block: four times the threads and a quarter of the
// instructions per thread and token, for a prompt of one or a few sequences, where the token-by-token chain of one
// (sequence, head) is what the step waits for and most of the GPU would idle.
template <bool ROW>
static int dispatch_scan(const ScanParams& p, int n_seqs, int max_new, cudaStream_t stream) {
  const int N = p.n_rows;
  const long narrow_blocks = (long)n_seqs * p.n_heads * ((p.n_cols + 15) / 16);
  const bool wide = max_new > 16 && narrow_blocks < 8l * sm_count() && N > 16 && N <= 256;
  if (wide) {
    // (one column per thread: a register tile of four columns per thread, which reads a row's k, q and decay once
    // for four columns, was measured slower at these sizes -- 4.7 against 2.7 ms for four layers of 2,048 tokens --
    // because it leaves a quarter of the threads and the token-by-token chain is what is waited for)
    // (sixteen lanes a column: thirty-two were measured slower, 5.0 against 2.7 ms for four layers of 2,048 tokens;
    // what a warp does per token besides its rows' arithmetic -- addresses, the value, the shuffle sum, the
    // store -- then weighs more than the rows.  Taking the shuffle sums of four tokens side by side changed
    // nothing: 2.6 ms.  Measured again with prepared decays and paired rows: 4.4 against 2.2 ms; twice the blocks
    // stage and read twice the rows of k, q and the decays.)
    if (N <= 64) return launch_scan<4, 16, ROW>(p, n_seqs, max_new, 8, stream);
    if (N <= 128) return launch_scan<8, 16, ROW>(p, n_seqs, max_new, 8, stream);
    if (N <= 192) return launch_scan<12, 16, ROW>(p, n_seqs, max_new, 8, stream);
    return launch_scan<16, 16, ROW>(p, n_seqs, max_new, 8, stream);
  }
  if (N <= 16) return launch_scan<4, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 32) return launch_scan<8, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 48) return launch_scan<12, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 64) return launch_scan<16, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 96) return launch_scan<24, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 128) return launch_scan<32, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 192) return launch_scan<48, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 256) return launch_scan<64, 4, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 512) return launch_scan<64, 8, ROW>(p, n_seqs, max_new, 2, stream);
  if (N <= 1024) return launch_scan<64, 16, ROW>(p, n_seqs, max_new, 2, stream);
  set_error("linear_scan: a state of %d rows per head is not supported (up to 1024)", N);
  return 1;
}


// ---- a gated linear recurrent unit with one state per channel --------------------------------------------------
//   r = sigmoid(g_r + b_r), i = sigmoid(g_i + b_i)          (g: the gates' block-diagonal products, computed before)
//   log a = -rate * softplus(lam) * r,   S_t = a S_{t-1} + sqrt(1 - a^2) * i * u_t,   out_t = S_t * gelu_tanh(y_t + b_y)
// all in float32; 1 - a^2 is taken as -expm1(2 log a), which keeps its digits when a is close to one.  A block takes
// `blockDim.x` (32, or 16 when that fills the GPU better) neighbouring channels of one sequence.  A step of many tokens
// is cut into `blockDim.y` runs of consecutive tokens: every run
// is first scanned from a zero state (its product of decays and what it adds), the runs' results are chained in
// shared memory, and a second pass repeats each run from its true entry state and writes the outputs.  A run of one
// thread row (decode, short portions) is the recurrence as written.
constexpr int RG_MAX_RUNS = 64;                   // with 16 channels a block; 32 with 32 (1,024 threads at most)

struct RgLruParams {
  const float* gates; long gates_stride; // [blocks * T, 2 * block]: row b * T + t = block b's gate rows of token t (r, then i)
  const void* r_bias; const void* i_bias; const void* lam; const void* y_bias; int small_dtype;      // [W] each; biases may be null
  const float* u; long u_stride;         // [T, W] the recurrence's input
  const float* y; long y_stride;         // [T, W] the other branch before its bias and activation
  float* state;                          // [slots, W]
  void* out; long out_stride;            // [T, W]
  const int* seq_slot; const int* seq_tok0; const int* seq_new;
  int n_tokens, width, block; float rate;
};

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TO>
__global__ void __launch_bounds__(1024) rglru_scan_kernel(RgLruParams p) {
  pdl_launch_dependents();
  __shared__ float A_s[RG_MAX_RUNS][32], B_s[RG_MAX_RUNS][32];
  const int tx = threadIdx.x, j = threadIdx.y, runs = blockDim.y;
  const int c = blockIdx.x * blockDim.x + tx, s = blockIdx.y;
  const bool live = c < p.width;
  float b_r = 0.f, b_i = 0.f, b_y = 0.f, rate = 0.f;
  if (live) {                                     // the channel's constants: no kernel writes them
    if (p.r_bias) b_r = load_any(p.r_bias, p.small_dtype, c);
    if (p.i_bias) b_i = load_any(p.i_bias, p.small_dtype, c);
    if (p.y_bias) b_y = load_any(p.y_bias, p.small_dtype, c);
    rate = -p.rate * softplus_f(load_any(p.lam, p.small_dtype, c));
  }
  pdl_wait();
  const int n = p.seq_new[s], tok0 = p.seq_tok0[s];
  const int len = (n + runs - 1) / runs;
  const int t_lo = min(n, j * len), t_hi = min(n, t_lo + len);
  const int cc = live ? c : 0;
  const float* g = p.gates + ((size_t)(cc / p.block) * p.n_tokens + tok0) * p.gates_stride + cc % p.block;
  const float* u = p.u + (size_t)tok0 * p.u_stride + cc;
  auto gate = [&](int t, float& a, float& x) {
    const float r = 1.0f / (1.0f + expf(-(g[(size_t)t * p.gates_stride] + b_r)));
    const float i = 1.0f / (1.0f + expf(-(g[(size_t)t * p.gates_stride + p.block] + b_i)));
    const float la = rate * r;
    a = expf(la);
    x = sqrtf(-expm1f(2.0f * la)) * (i * u[(size_t)t * p.u_stride]);
  };
  if (runs > 1) {
    float A = 1.f, B = 0.f;
    if (live) {
#pragma unroll 4
      for (int t = t_lo; t < t_hi; ++t) {
        float a, x;
        gate(t, a, x);
        B = fmaf(a, B, x);
        A *= a;
      }
    }
    A_s[j][tx] = A; B_s[j][tx] = B;
    __syncthreads();
  }
  if (!live) return;
  float* st = p.state + (size_t)p.seq_slot[s] * p.width + c;
  float S = *st;
  for (int jj = 0; jj < j; ++jj) S = fmaf(A_s[jj][tx], S, B_s[jj][tx]);
  const float* y = p.y + (size_t)tok0 * p.y_stride + c;
  TO* o = reinterpret_cast<TO*>(p.out) + (size_t)tok0 * p.out_stride + c;
#pragma unroll 4
  for (int t = t_lo; t < t_hi; ++t) {
    float a, x;
    gate(t, a, x);
    S = fmaf(a, S, x);
    o[(size_t)t * p.out_stride] = from_f32<TO>(S * gelu_tanh_f(y[(size_t)t * p.y_stride] + b_y));
  }
  if (j == runs - 1) *st = S;                      // the last run's exit state is the sequence's (an empty run passes it on)
}


// out[b * T + t, :] = in[t, b * n : (b + 1) * n] in out's dtype: the equal parts of float32 rows laid out part by part,
// as the rows of a grouped product with one group per part; offsets[b] = b * T for b = 0 .. parts.
template <typename TO>
__global__ void __launch_bounds__(256) block_major_rows_kernel(const float* __restrict__ in, long in_stride,
                                                               TO* __restrict__ out, int* __restrict__ offsets,
                                                               int n_tokens, int parts, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* src = in + (size_t)t * in_stride;
  for (int i = threadIdx.x; i < parts * n; i += blockDim.x)
    out[((size_t)(i / n) * n_tokens + t) * n + i % n] = from_f32<TO>(src[i]);
  if (t == 0)
    for (int b = threadIdx.x; b <= parts; b += blockDim.x) offsets[b] = b * n_tokens;
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_block_major_rows(const float* in, long in_stride, void* out, int out_dtype, int* offsets,
                                    int n_tokens, int parts, int n, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(parts >= 1 && n >= 1, "block_major_rows: %d parts of %d elements", parts, n);
  CPI_DISPATCH_DTYPE(out_dtype, TO, cpi::launch_pdl(block_major_rows_kernel<TO>, dim3(n_tokens), dim3(256), 0, stream, in,
                                                    in_stride, reinterpret_cast<TO*>(out), offsets, n_tokens, parts, n));
  return check_launch("block_major_rows");
}

extern "C" int cpi_rglru_scan(const float* gates, long gates_stride, const void* r_bias, const void* i_bias,
                              const void* lam, const void* y_bias, int small_dtype, const float* u, long u_stride,
                              const float* y, long y_stride, float* state, void* out, int out_dtype, long out_stride,
                              const int* seq_slot, const int* seq_tok0, const int* seq_new, int n_seqs, int max_new,
                              int n_tokens, int width, int block, float rate, cudaStream_t stream) {
  if (n_seqs == 0 || n_tokens == 0) return 0;
  CPI_REQUIRE(width > 0 && block > 0 && width % block == 0, "rglru_scan: %d channels in blocks of %d", width, block);
  CPI_REQUIRE(lam != nullptr, "rglru_scan: the channels' decay parameters are missing");
  CPI_REQUIRE(n_seqs <= 65535, "rglru_scan: too many sequences in one step (%d)", n_seqs);
  RgLruParams p{gates, gates_stride, r_bias, i_bias, lam, y_bias, small_dtype, u, u_stride, y, y_stride, state, out,
                out_stride, seq_slot, seq_tok0, seq_new, n_tokens, width, block, rate};
  // runs of at least 16 tokens, as many as fill the GPU twice over; 16 channels a block (64-byte segments) where 32
  // would leave SMs without a block
  int runs = 1, ch = 32;
  if (max_new >= 32) {
    if (n_seqs * ((width + 31) / 32) < 2 * sm_count()) ch = 16;
    const int blocks = n_seqs * ((width + ch - 1) / ch);
    runs = (2 * sm_count() * 2048 / ch + blocks - 1) / blocks;
    if (runs > max_new / 16) runs = max_new / 16;
    if (runs > 1024 / ch) runs = 1024 / ch;
    if (runs < 1) runs = 1;
  }
  const dim3 grid((width + ch - 1) / ch, n_seqs), block_dim(ch, runs);
  CPI_DISPATCH_DTYPE(out_dtype, TO, cpi::launch_pdl(rglru_scan_kernel<TO>, grid, block_dim, 0, stream, p));
  return check_launch("rglru_scan");
}

extern "C" int cpi_causal_conv(const float* in, long in_stride, const void* w, const void* bias, int w_dtype,
                               float* carry, const int* token_seq, const int* token_pos, const int* seq_slot,
                               const int* seq_start, const int* seq_tok0, const int* seq_new, float* out,
                               long out_stride, int n_tokens, int n_seqs, int channels, int taps, int silu,
                               const void* in_bias, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: %d taps (supported: 1 to %d)", taps, CONV_MAX_TAPS);
  CPI_REQUIRE(channels > 0 && n_seqs > 0, "causal_conv: bad sizes C=%d sequences=%d", channels, n_seqs);
  ConvParams p{in, in_stride, w, bias, w_dtype, carry, token_seq, token_pos, seq_slot, seq_start, seq_tok0, seq_new,
               out, out_stride, channels, taps, silu, in_bias};
  const int threads = channels <= 128 ? 128 : 256;
  cpi::launch_pdl(causal_conv_kernel, dim3(n_tokens, (channels + threads - 1) / threads), threads, 0, stream, p);
  if (int rc = check_launch("causal_conv")) return rc;
  if (taps > 1) {
    cpi::launch_pdl(conv_carry_kernel, dim3(n_seqs, (channels + threads - 1) / threads), threads, 0, stream, p);
    return check_launch("conv_carry");
  }
  return 0;
}

extern "C" int cpi_linear_scan(const float* k, long k_stride, const float* q, long q_stride, const float* v,
                               long v_stride, const float* z, long z_stride, const void* z_bias, float inv_tau,
                               const float* dt, long dt_stride, const void* dt_bias, const void* a_log,
                               const void* skip, int small_dtype, float q_scale, float* state, float* out,
                               long out_stride, const int* seq_slot, const int* seq_tok0, const int* seq_new,
                               int n_seqs, int max_new, int n_heads, int heads_per_group, int n_rows, int n_cols,
                               int decay_ready, int decay_kind, const float* beta, long beta_stride,
                               cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CPI_REQUIRE((z != nullptr) != (dt != nullptr), "linear_scan: give row decays or step sizes, one of the two");
  CPI_REQUIRE(dt == nullptr || a_log != nullptr, "linear_scan: step sizes need the heads' decay rates");
  CPI_REQUIRE(n_heads > 0 && heads_per_group > 0 && n_heads % heads_per_group == 0 && n_rows > 0 && n_cols > 0,
              "linear_scan: bad sizes heads=%d per group=%d rows=%d columns=%d", n_heads, heads_per_group, n_rows, n_cols);
  CPI_REQUIRE(n_heads <= 65535, "linear_scan: too many heads (%d)", n_heads);
  CPI_REQUIRE(decay_kind == 0 || (decay_kind == 1 && z != nullptr && a_log != nullptr),
              "linear_scan: decay kind %d needs row decays and the heads' rates", decay_kind);
  CPI_REQUIRE(beta == nullptr || z != nullptr, "linear_scan: the delta rule comes with row decays");
  ScanParams p{k, k_stride, q, q_stride, v, v_stride, z, z_stride, z_bias, inv_tau, dt, dt_stride, dt_bias, a_log,
               skip, small_dtype, q_scale, state, out, out_stride, seq_slot, seq_tok0, seq_new,
               n_heads, heads_per_group, n_rows, n_cols, 0, 0, decay_ready, decay_kind, beta, beta_stride};
  if (max_new < 1) max_new = 1;
  return z ? dispatch_scan<true>(p, n_seqs, max_new, stream) : dispatch_scan<false>(p, n_seqs, max_new, stream);
}

extern "C" int cpi_row_decay(float* z, long z_stride, const void* bias, int bias_dtype, float inv_tau, int n_tokens,
                             int n, int kind, const void* a_log, int rows_per_head, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n > 0, "row_decay: %d elements a row", n);
  CPI_REQUIRE(kind == 0 || (kind == 1 && a_log != nullptr && rows_per_head > 0), "row_decay: kind %d needs the heads' rates", kind);
  RowDecayParams p{z, z_stride, bias, bias_dtype, inv_tau, n, kind, a_log, rows_per_head};
  cpi::launch_pdl(row_decay_kernel, dim3(n_tokens, (n + 255) / 256), 256, 0, stream, p);
  return check_launch("row_decay");
}

extern "C" int cpi_gated_norm(const float* y, long y_stride, const float* gate, long gate_stride, const void* w,
                              int w_dtype, int w_len, void* out, int out_dtype, long out_stride, int n_tokens,
                              int width, int parts, int gate_first, float eps, int gate_act, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(width > 0 && parts > 0 && width % parts == 0, "gated_norm: %d elements in %d parts", width, parts);
  CPI_REQUIRE(parts <= 65535, "gated_norm: too many parts (%d)", parts);
  CPI_REQUIRE(!w || w_len > 0, "gated_norm: a weight needs a length");
  CPI_REQUIRE(gate_act == 0 || gate_act == 1, "gated_norm: unknown gate activation %d", gate_act);
  GatedNormParams p{y, y_stride, gate, gate_stride, w, w_dtype, w_len, out, out_stride, width, parts, gate_first, eps, gate_act};
  CPI_DISPATCH_DTYPE(out_dtype, TO, cpi::launch_pdl(gated_norm_kernel<TO>, dim3(n_tokens, parts), 128, 0, stream, p));
  return check_launch("gated_norm");
}

extern "C" int cpi_head_unit(float* x, long stride, int n_tokens, int heads, int dim, float eps, cudaStream_t stream) {
  if (n_tokens == 0 || heads == 0) return 0;
  CPI_REQUIRE(heads > 0 && dim > 0, "head_unit: %d heads of %d elements", heads, dim);
  cpi::launch_pdl(head_unit_kernel, dim3(n_tokens, (heads + 3) / 4), 128, 0, stream, x, stride, heads, dim, eps);
  return check_launch("head_unit");
}
