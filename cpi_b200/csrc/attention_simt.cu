// Attention over the paged key/value cache, general form: any head size up to 256, any number of heads
// and groups, float32 or bfloat16, prompts and single tokens alike.
//
//   qkv_post     per token and head: optional weightless RMS norm of q and k, rotary position encoding,
//                optional query temperature; writes q to its buffer and k, v into the cache pages
//                (head sizes that are multiples of 16).
//   qkv_prepare  the same step for mixers with biases, an RMS norm over the whole q and the whole k projection
//                (with weights), a rotation of only the first elements of each head, or values of another size
//                than keys, or a weightless RMS norm of every q and k head after the rotation; a block per token,
//                float32 or bfloat16 rows in.
//                Also: two score maps per head (second halves of the q and k rows to buffers of their own), values that
//                are the projected keys, a query temperature, an amplitude on the rotation.
//   head_post    what follows attention per token and head: a1 - lambda a2, its weightless norm, a sigmoid gate.
//   attention    one block per (token, head): scores over the keys the window allows, softmax and the
//                weighted sum of values in float32, keys visited in position order.  A position encoding
//                that acts on the scores hands in a table: score(query at p, key at t) += bias[head][min(p - t,
//                n_dist - 1)].  A sink (a number per head) joins the softmax denominator as exp(sink), with no
//                key and no value.  Values may have another size than keys.
//
// Formulas (file:line of kurulav1/cpi): per-head norm src/engine/llama4_cpu_engine.cpp:308-317; RoPE pairs
// (d, d + D/2) with angle float(p) * theta_d :167-193, :467; scores, softmax with 1/max(sum, 1e-20) and
// value sum :195-250.  Windows, layers without RoPE, interleaved pairing and the query temperature
// q *= 1 + a * ln(floor((p + 1) / f) + 1) are this library's own.  A sliding window may keep a sequence's first
// `keep_first` positions visible to every later query (at their own positions), whatever the distance.
//
// Cache layout per layer: [page][kv head][slot in page][D]; a sequence's block b (positions
// b*PAGE .. b*PAGE+PAGE-1) lives in page page_table[slot * max_blocks + b].
#include "common.cuh"

namespace cpi {

struct QkvPostParams {
  const void* qkv; long qkv_stride;      // [T, (NH + 2 NKV) D]   (or [T, NH D] when write_kv == 0)
  void* q_out;                           // [T, NH D]
  void* k_cache; void* v_cache;
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  const float* inv_freq;                 // [D/2] or null: no rotation
  int interleaved;
  int qk_norm; int norm_before_rope; float norm_eps;
  int temperature; float floor_scale; float attn_scale;
  int n_heads, n_kv_heads, head_dim, write_kv;
};

template <typename T>
__global__ void qkv_post_kernel(QkvPostParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = p.n_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int hs = blockIdx.y * (blockDim.x >> 5) + warp;       // head slot
  if (hs >= heads_total) return;
  const int t = blockIdx.x;
  const int D = p.head_dim, half = D >> 1;
  const T* src = reinterpret_cast<const T*>(p.qkv) + (size_t)t * p.qkv_stride + (size_t)hs * D;
  const int pos = p.token_pos[t];
  const bool is_q = hs < p.n_heads;
  const bool is_v = hs >= p.n_heads + p.n_kv_heads;

  T* dst;
  if (is_q) {
    dst = reinterpret_cast<T*>(p.q_out) + ((size_t)t * p.n_heads + hs) * D;
  } else {
    const int kvh = is_v ? hs - p.n_heads - p.n_kv_heads : hs - p.n_heads;
    const int slot = p.seq_slot[p.token_seq[t]];
    const int page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
    T* base = reinterpret_cast<T*>(is_v ? p.v_cache : p.k_cache);
    dst = base + (((size_t)page * p.n_kv_heads + kvh) * p.page_size + pos % p.page_size) * D;
  }
  if (is_v) {
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  float a[4], b[4];                      // pairs lane, lane+32, ... (D <= 256)
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    a[j] = b[j] = 0.f;
    if (i < half) {
      const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
      a[j] = to_f32(src[ia]); b[j] = to_f32(src[ib]);
      ss += a[j] * a[j] + b[j] * b[j];
    }
  }
  if (p.qk_norm && p.norm_before_rope) {
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.norm_eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= inv; b[j] *= inv; }
  }
  if (p.inv_freq) {
    ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        const float ang = (float)pos * p.inv_freq[i];
        float s, c;
        sincosf(ang, &s, &c);
        const float x = a[j], y = b[j];
        a[j] = x * c - y * s;
        b[j] = x * s + y * c;
        ss += a[j] * a[j] + b[j] * b[j];
      }
    }
  }
  if (p.qk_norm && !p.norm_before_rope) {
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.norm_eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= inv; b[j] *= inv; }
  }
  if (is_q && p.temperature) {
    const float sc = 1.0f + p.attn_scale * logf(floorf(((float)pos + 1.0f) / p.floor_scale) + 1.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= sc; b[j] *= sc; }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
      dst[ia] = from_f32<T>(a[j]); dst[ib] = from_f32<T>(b[j]);
    }
  }
}

// The same work for bfloat16 heads of 128 with half-split pairs, 16 bytes per lane: a warp takes two heads
// at a time (lanes 0-15 one, 16-31 the other; lane l of a head holds elements 8l .. 8l+7, its rotation
// partner sits 8 lanes away), a block takes a slice of one token's heads and computes the token's 64
// sines and cosines once.  Same formulas as qkv_post_kernel; sums of squares in another order.
__global__ void __launch_bounds__(256) qkv_post_d128_kernel(QkvPostParams p, int heads_per_block) {
  __shared__ float cos_s[64], sin_s[64];
  pdl_launch_dependents();
  // positions and page tables are copied to the device before the step's first kernel and the frequencies
  // are constants: the angles do not wait for the kernel that writes q, k and v
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = p.token_pos[t];
  if (p.inv_freq && tid < 64) {
    float s, c;
    sincosf((float)pos * p.inv_freq[tid], &s, &c);
    cos_s[tid] = c; sin_s[tid] = s;
  }
  pdl_wait();
  __syncthreads();
  const int heads_total = p.n_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int h_begin = blockIdx.y * heads_per_block, h_end = min(heads_total, h_begin + heads_per_block);
  const int sub = lane >> 4, l = lane & 15;
  const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(p.qkv) + (size_t)t * p.qkv_stride;
  int page = 0;
  if (p.write_kv) {
    const int slot = p.seq_slot[p.token_seq[t]];
    page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
  }
  const float temp = p.temperature ? 1.0f + p.attn_scale * logf(floorf(((float)pos + 1.0f) / p.floor_scale) + 1.0f) : 1.0f;
  for (int hs = h_begin + 2 * warp + sub; hs < h_end + sub; hs += 2 * (blockDim.x >> 5)) {
    // (all 32 lanes stay in the loop together so that the shuffles below are whole-warp; a lane whose
    // head is past the end computes on zeros and stores nothing)
    const bool live = hs < h_end;
    const bool is_q = hs < p.n_heads, is_v = hs >= p.n_heads + p.n_kv_heads;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = *reinterpret_cast<const uint4*>(row + (size_t)hs * 128 + 8 * l);
    __nv_bfloat16* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = reinterpret_cast<__nv_bfloat16*>(p.q_out) + ((size_t)t * p.n_heads + hs) * 128 + 8 * l;
      } else {
        const int kvh = is_v ? hs - p.n_heads - p.n_kv_heads : hs - p.n_heads;
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? p.v_cache : p.k_cache);
        dst = base + (((size_t)page * p.n_kv_heads + kvh) * p.page_size + pos % p.page_size) * 128 + 8 * l;
      }
    }
    float x[8];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); x[2 * j] = f.x; x[2 * j + 1] = f.y; }
    }
    const bool rotate = !is_v;                                  // v is copied as it is
    auto group_sum = [&](float v) {
      v += __shfl_xor_sync(0xffffffffu, v, 8); v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 1);
      return v;
    };
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    ss = group_sum(ss);
    if (p.qk_norm && p.norm_before_rope && rotate) {
      const float inv = 1.0f / sqrtf(ss / 128.0f + p.norm_eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= inv;
    }
    if (p.inv_freq) {
      float other[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) other[j] = __shfl_xor_sync(0xffffffffu, x[j], 8);
      if (rotate) {
        const bool first = l < 8;                               // first half: a' = a c - b s; second: b' = a s + b c
        ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = 8 * (l & 7) + j;
          const float c = cos_s[i], sn = sin_s[i];
          x[j] = first ? x[j] * c - other[j] * sn : other[j] * sn + x[j] * c;
          ss += x[j] * x[j];
        }
      }
      ss = group_sum(ss);
    }
    if (p.qk_norm && !p.norm_before_rope && rotate) {
      const float inv = 1.0f / sqrtf(ss / 128.0f + p.norm_eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= inv;
    }
    if (is_q && p.temperature) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= temp;
    }
    if (live) {
      uint4 o;
      if (is_v) {
        o = raw;
      } else {
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
      }
      *reinterpret_cast<uint4*>(dst) = o;
    }
  }
}

// The same step in its general form, a block per token: biases, an RMS norm over the whole q projection and the
// whole k projection (all heads at once, with weights), a rotation of only the first `rot_dims` elements of each
// head (pairs (i, i + rot_dims / 2); the rest pass), values of another size than keys.  Input rows may be float32
// while the cache is bfloat16: the row is then rounded once, after the norm and the rotation.
struct QkvPrepParams {
  const void* qkv; long qkv_stride;      // [T, NH D + NKV D + NKV DV]
  const void* bias; int bias_dtype;      // [NH D + NKV D + NKV DV] or null
  const void* q_norm; const void* k_norm; int norm_dtype; int norm_whole; float norm_eps;     // weights or null
  const float* inv_freq; int rot_dims;   // [rot_dims / 2] or null
  void* q_out; void* k_cache; void* v_cache;
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  int n_heads, n_kv_heads, head_dim, v_dim, write_kv;
  int head_norm;                         // 1: a weightless RMS norm (norm_eps) of every q and k head, after the rotation;
                                         // 2: an RMS norm of every q and k head before the rotation, times q_norm / k_norm
                                         //    ([head_dim] each, shared by the heads; null: no weight)
  int interleaved;                       // the rotation pairs elements (2i, 2i + 1) instead of (i, i + rot_dims / 2)
  float* v_first; long v_first_stride;   // value mixing (float32 [T, NKV DV]): v_mix_mode 1 stores this layer's values
  const void* v_mix; int v_mix_dtype;    // there; 2 writes v <- (1 - m) v + m v_first[t] with the one number m = *v_mix
  int v_mix_mode;
  int maps;                              // 1, or 2: q rows hold 2 NH heads and k rows 2 NKV heads, the second halves being the
  void* q2_out; void* k2_cache;          // heads of a second score map, which go to q2_out and k2_cache (shaped like the first)
  int v_from_k;                          // the values are the k rows as projected (bias added, before any norm); rows hold no v
  int temperature; float floor_scale; float attn_scale;      // q *= 1 + attn_scale * ln(floor((pos + 1) / floor_scale) + 1)
  float rot_amp;                         // the sines and cosines of the rotation are multiplied by this
};

// which element a rotated element d is paired with, whether it is the pair's first, and the pair's frequency index
__device__ __forceinline__ void rot_pair(int d, int half, int interleaved, bool& first, int& other, int& f) {
  if (interleaved) { first = !(d & 1); other = d ^ 1; f = d >> 1; }
  else { first = d < half; other = first ? d + half : d - half; f = first ? d : d - half; }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(1024) qkv_prepare_kernel(QkvPrepParams p) {
  pdl_launch_dependents();
  extern __shared__ float row_s[];                       // q then k of this token, float32
  __shared__ float scratch[32];
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int D = p.head_dim, DV = p.v_dim;
  const int nq = p.maps * p.n_heads * D, nk = p.write_kv ? p.maps * p.n_kv_heads * D : 0, nv = p.write_kv ? p.n_kv_heads * DV : 0;
  const TI* src = reinterpret_cast<const TI*>(p.qkv) + (size_t)t * p.qkv_stride;
  const int pos = p.token_pos[t];
  const float temp = p.temperature ? 1.0f + p.attn_scale * logf(floorf(((float)pos + 1.0f) / p.floor_scale) + 1.0f) : 1.0f;
  // a step of few tokens is also cut along the heads: block (t, y) takes the q and k heads [h0, h1) of the row and the
  // value heads [vh0, vh1) (one slice when the norm runs over the whole projection)
  const int heads_all = (nq + nk) / D, v_heads = nv / DV;
  const int h0 = (int)((long)heads_all * blockIdx.y / gridDim.y), h1 = (int)((long)heads_all * (blockIdx.y + 1) / gridDim.y);
  const int e0 = h0 * D, e1 = h1 * D;
  const int v0 = (int)((long)v_heads * blockIdx.y / gridDim.y) * DV, v1 = (int)((long)v_heads * (blockIdx.y + 1) / gridDim.y) * DV;
  float ssq = 0.f, ssk = 0.f;
  for (int i = e0 + tid; i < e1; i += blockDim.x) {
    float x = to_f32(src[i]);
    if (p.bias) x += load_any(p.bias, p.bias_dtype, i);
    row_s[i] = x;
    if (i < nq) ssq = fmaf(x, x, ssq); else ssk = fmaf(x, x, ssk);
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (p.norm_whole) {
    ssq = block_sum(ssq, scratch);
    inv_q = 1.0f / sqrtf(ssq / (float)nq + p.norm_eps);
    if (nk) {
      ssk = block_sum(ssk, scratch);
      inv_k = 1.0f / sqrtf(ssk / (float)nk + p.norm_eps);
    }
  }
  __syncthreads();
  size_t kv_row = 0;
  if (p.write_kv) {
    const int slot = p.seq_slot[p.token_seq[t]];
    const int page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
    kv_row = (size_t)page * p.n_kv_heads * p.page_size + pos % p.page_size;      // row of kv head 0
  }
  // element i of the q part / element e of the k part, to the first map's buffer or the second's
  auto store_q = [&](int i, float x) {
    const int hd = i / D;
    TO* base = reinterpret_cast<TO*>(hd < p.n_heads ? p.q_out : p.q2_out);
    base[((size_t)t * p.n_heads + hd % p.n_heads) * D + i % D] = from_f32<TO>(x * temp);
  };
  auto store_k = [&](int e, float x) {
    const int hd = e / D;
    TO* base = reinterpret_cast<TO*>(hd < p.n_kv_heads ? p.k_cache : p.k2_cache);
    base[(kv_row + (size_t)(hd % p.n_kv_heads) * p.page_size) * D + e % D] = from_f32<TO>(x);
  };
  const int half = p.rot_dims >> 1;
  float* rot_s = row_s + nq + nk;                        // head_norm: the rotated row, then one factor per head
  float* inv_s = rot_s + nq + nk;
  if (p.head_norm == 1) {
    for (int i = e0 + tid; i < e1; i += blockDim.x) {
      const int e = i < nq ? i : i - nq, d = e % D;
      float x = row_s[i];
      if (p.inv_freq && d < p.rot_dims) {
        bool first; int od, f;
        rot_pair(d, half, p.interleaved, first, od, f);
        const float other = row_s[i - d + od];
        float sn, cs;
        sincosf((float)pos * p.inv_freq[f], &sn, &cs);
        sn *= p.rot_amp; cs *= p.rot_amp;
        x = first ? x * cs - other * sn : x * cs + other * sn;
      }
      rot_s[i] = x;
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    for (int hd = h0 + warp; hd < h1; hd += blockDim.x >> 5) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss = fmaf(rot_s[hd * D + d], rot_s[hd * D + d], ss);
      ss = warp_sum(ss);
      if (lane == 0) inv_s[hd] = 1.0f / sqrtf(ss / (float)D + p.norm_eps);
    }
    __syncthreads();
    for (int i = e0 + tid; i < e1; i += blockDim.x) {
      const bool is_q = i < nq;
      const int e = is_q ? i : i - nq;
      const float x = rot_s[i] * inv_s[i / D];
      if (is_q) store_q(i, x);
      else store_k(e, x);
    }
  }
  if (p.head_norm == 2) {
    // every head by its own root mean square, times the weight of its element, and then the rotation
    float* inv_h = row_s + nq + nk;
    const int warp = tid >> 5, lane = tid & 31;
    for (int hd = h0 + warp; hd < h1; hd += blockDim.x >> 5) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss = fmaf(row_s[hd * D + d], row_s[hd * D + d], ss);
      ss = warp_sum(ss);
      if (lane == 0) inv_h[hd] = 1.0f / sqrtf(ss / (float)D + p.norm_eps);
    }
    __syncthreads();
    for (int i = e0 + tid; i < e1; i += blockDim.x) {
      const bool is_q = i < nq;
      const int e = is_q ? i : i - nq;
      const int hd = e / D, d = e % D;
      const void* nw = is_q ? p.q_norm : p.k_norm;
      const float inv = inv_h[i / D];
      auto normed = [&](int idx, int el) {
        float x = row_s[idx] * inv;
        if (nw) x *= load_any(nw, p.norm_dtype, el);
        return x;
      };
      float x = normed(i, d);
      if (p.inv_freq && d < p.rot_dims) {
        bool first; int od, f;
        rot_pair(d, half, p.interleaved, first, od, f);
        const float other = normed(i - d + od, od);
        float sn, cs;
        sincosf((float)pos * p.inv_freq[f], &sn, &cs);
        sn *= p.rot_amp; cs *= p.rot_amp;
        x = first ? x * cs - other * sn : x * cs + other * sn;
      }
      if (is_q) store_q(i, x);
      else store_k(e, x);
    }
  }
  for (int i = e0 + tid; i < (p.head_norm ? 0 : e1); i += blockDim.x) {
    const bool is_q = i < nq;
    const int e = is_q ? i : i - nq;
    const int hd = e / D, d = e % D;
    const float inv = is_q ? inv_q : inv_k;
    const void* nw = is_q ? p.q_norm : p.k_norm;
    auto normed = [&](int idx, int el) {
      float x = row_s[idx] * inv;
      if (p.norm_whole && nw) x *= load_any(nw, p.norm_dtype, el);
      return x;
    };
    float x = normed(i, e);
    if (p.inv_freq && d < p.rot_dims) {
      bool first; int od, f;
      rot_pair(d, half, p.interleaved, first, od, f);
      const float other = normed(i - d + od, e - d + od);
      float sn, cs;
      sincosf((float)pos * p.inv_freq[f], &sn, &cs);
      sn *= p.rot_amp; cs *= p.rot_amp;
      x = first ? x * cs - other * sn : x * cs + other * sn;
    }
    if (is_q) store_q(i, x);
    else store_k(e, x);
  }
  for (int i = v0 + tid; i < v1; i += blockDim.x) {
    float x;
    if (p.v_from_k) {                                    // the key as projected, its bias added, before the norm
      x = to_f32(src[nq + i]);
      if (p.bias) x += load_any(p.bias, p.bias_dtype, nq + i);
    } else {
      x = to_f32(src[nq + nk + i]);
      if (p.bias) x += load_any(p.bias, p.bias_dtype, nq + nk + i);
    }
    if (p.v_mix_mode == 1) {
      p.v_first[(size_t)t * p.v_first_stride + i] = x;
    } else if (p.v_mix_mode == 2) {
      const float m = load_any(p.v_mix, p.v_mix_dtype, 0);
      x = (1.0f - m) * x + m * p.v_first[(size_t)t * p.v_first_stride + i];
    }
    reinterpret_cast<TO*>(p.v_cache)[(kv_row + (size_t)(i / DV) * p.page_size) * DV + i % DV] = from_f32<TO>(x);
  }
}

struct AttnParams {
  const void* q; void* out;              // [T, NH D]
  const void* k_cache; const void* v_cache;
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  int n_heads, n_kv_heads, head_dim;
  int window_kind, window_size;          // 0 all keys, 1 chunk of window_size, 2 last window_size keys
  float scale;
  const float* score_bias; int n_dist;   // [NH, n_dist] float32 added to the scaled scores by distance, or null
  const float* sink;                     // [NH] float32 or null: exp(sink[h]) joins the softmax denominator (no key, no value)
  int v_dim;                             // elements of a value row (the cache's v stream); keys have head_dim
  int keep_first;                        // a sequence's first positions that stay visible below a sliding window
  float softcap;                         // > 0: score <- softcap * tanh(score / softcap) after the scale
};

__device__ __forceinline__ int window_low(int kind, int size, int pos) {
  if (kind == 1) return (pos / size) * size;
  if (kind == 2) return max(0, pos - size + 1);
  return 0;
}

constexpr int ATT_NT = 128;
constexpr int ATT_MAX_DIM = 640;                 // the largest key or value row: ATT_ACC accumulators per thread
constexpr int ATT_ACC = ATT_MAX_DIM / ATT_NT;

template <typename T>
__global__ void __launch_bounds__(ATT_NT) attention_general_kernel(AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float q_s[ATT_MAX_DIM];
  __shared__ float p_s[ATT_NT];
  __shared__ size_t off_s[ATT_NT];
  __shared__ float scratch[32];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int D = p.head_dim, DV = p.v_dim;
  const int kvh = h / (p.n_heads / p.n_kv_heads);
  const int pos = p.token_pos[t];
  const int slot = p.seq_slot[p.token_seq[t]];
  const int lo = window_low(p.window_kind, p.window_size, pos);
  const T* q = reinterpret_cast<const T*>(p.q) + ((size_t)t * p.n_heads + h) * D;
  for (int i = tid; i < D; i += ATT_NT) q_s[i] = to_f32(q[i]);
  const T* kc = reinterpret_cast<const T*>(p.k_cache);
  const T* vc = reinterpret_cast<const T*>(p.v_cache);
  const int* table = p.page_table + (size_t)slot * p.max_blocks;

  // a sink is a key without a value whose score is sink[h], unscaled: the running maximum and sum start from it
  float m_run = -INFINITY, l_run = 0.f;
  float acc[ATT_ACC];
#pragma unroll
  for (int a = 0; a < ATT_ACC; ++a) acc[a] = 0.f;
  if (p.sink) { m_run = p.sink[h]; l_run = 1.0f; }
  __syncthreads();
  // the keys a query sees: the kept first positions that lie below the window, then the window
  const int n_kept = min(p.keep_first, lo), n_keys = n_kept + pos - lo + 1;
  for (int base = 0; base < n_keys; base += ATT_NT) {
    const int ki = base + tid;
    const int kp = ki < n_kept ? ki : lo + ki - n_kept;
    const bool valid = ki < n_keys;
    float s = -INFINITY;
    if (valid) {
      const int page = table[kp / p.page_size];
      const size_t row = ((size_t)page * p.n_kv_heads + kvh) * p.page_size + kp % p.page_size;
      off_s[tid] = row;
      const T* kr = kc + row * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(q_s[d], to_f32(kr[d]), dot);
      s = dot * p.scale;
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
      if (p.score_bias) s += p.score_bias[(size_t)h * p.n_dist + min(pos - kp, p.n_dist - 1)];
    }
    const float m_new = fmaxf(m_run, block_max(s, scratch));
    const float e = valid ? expf(s - m_new) : 0.f;
    p_s[tid] = e;
    const float l_tile = block_sum(e, scratch);       // its barriers also publish p_s and off_s
    const float alpha = expf(m_run - m_new);
    const int nv = min(ATT_NT, n_keys - base);
#pragma unroll
    for (int a = 0; a < ATT_ACC; ++a) acc[a] *= alpha;
    for (int j = 0; j < nv; ++j) {
      const T* vr = vc + off_s[j] * DV;
      const float pj = p_s[j];
#pragma unroll
      for (int a = 0; a < ATT_ACC; ++a)
        if (tid + a * ATT_NT < DV) acc[a] = fmaf(pj, to_f32(vr[tid + a * ATT_NT]), acc[a]);
    }
    l_run = l_run * alpha + l_tile;
    m_run = m_new;
    __syncthreads();
  }
  const float inv = 1.0f / fmaxf(l_run, 1e-20f);
  T* o = reinterpret_cast<T*>(p.out) + ((size_t)t * p.n_heads + h) * DV;
#pragma unroll
  for (int a = 0; a < ATT_ACC; ++a)
    if (tid + a * ATT_NT < DV) o[tid + a * ATT_NT] = from_f32<T>(acc[a] * inv);
}

// What follows attention, per token and head, before the output projection (one warp a head):
//   o = a1 - lambda * a2        (a2: the output of a second score map over the same values; null: o = a1)
//   o <- o / sqrt(mean(o^2) + eps) * norm_scale      (when `norm`: over the head's values, no weight)
//   o <- o * sigmoid(gate[t, h])                     (when `gate`: one number per token and head, float32 before its sigmoid)
// in float32, rounded once into `out` (which may be a1).
struct HeadPostParams {
  const void* a1; const void* a2; void* out;             // [T, NH * DV]
  float lambda; int norm; float eps; float norm_scale;
  const float* gate; long gate_stride;
  int n_tokens, n_heads, v_dim;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(128) head_post_kernel(HeadPostParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long r = (long)blockIdx.x * (blockDim.x >> 5) + warp;           // (token, head)
  if (r >= (long)p.n_tokens * p.n_heads) return;
  const int t = (int)(r / p.n_heads), h = (int)(r % p.n_heads);
  const int DV = p.v_dim;
  const TI* a1 = reinterpret_cast<const TI*>(p.a1) + (size_t)r * DV;
  const TI* a2 = p.a2 ? reinterpret_cast<const TI*>(p.a2) + (size_t)r * DV : nullptr;
  TO* o = reinterpret_cast<TO*>(p.out) + (size_t)r * DV;
  float f = 1.0f;
  if (p.norm) {
    float ss = 0.f;
    for (int d = lane; d < DV; d += 32) {
      const float x = a2 ? to_f32(a1[d]) - p.lambda * to_f32(a2[d]) : to_f32(a1[d]);
      ss = fmaf(x, x, ss);
    }
    f = p.norm_scale / sqrtf(warp_sum(ss) / (float)DV + p.eps);
  }
  if (p.gate) f *= 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.gate_stride + h]));
  for (int d = lane; d < DV; d += 32) {
    const float x = a2 ? to_f32(a1[d]) - p.lambda * to_f32(a2[d]) : to_f32(a1[d]);
    o[d] = from_f32<TO>(x * f);
  }
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_head_post(const void* a1, const void* a2, int in_dtype, void* out, int out_dtype, float lambda,
                             int norm, float eps, float norm_scale, const float* gate, long gate_stride, int n_tokens,
                             int n_heads, int v_dim, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_heads > 0 && v_dim > 0, "head_post: %d heads of %d values", n_heads, v_dim);
  HeadPostParams p{a1, a2, out, lambda, norm, eps, norm_scale, gate, gate_stride, n_tokens, n_heads, v_dim};
  const long rows = (long)n_tokens * n_heads;
  const dim3 grid((unsigned)((rows + 3) / 4));
  if (in_dtype == kF32 && out_dtype == kF32) cpi::launch_pdl(head_post_kernel<float, float>, grid, 128, 0, stream, p);
  else if (in_dtype == kF32 && out_dtype == kBF16) cpi::launch_pdl(head_post_kernel<float, __nv_bfloat16>, grid, 128, 0, stream, p);
  else if (in_dtype == kBF16 && out_dtype == kBF16) cpi::launch_pdl(head_post_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 128, 0, stream, p);
  else { set_error("head_post: input dtype %d with output dtype %d is not supported", in_dtype, out_dtype); return 1; }
  return check_launch("head_post");
}

static int check_head(const char* who, int n_heads, int n_kv_heads, int head_dim) {
  CPI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
              "%s: %d heads cannot be grouped over %d key/value heads", who, n_heads, n_kv_heads);
  CPI_REQUIRE(head_dim >= 16 && head_dim <= 256 && head_dim % 16 == 0,
              "%s: head size %d is not supported (multiples of 16 from 16 to 256)", who, head_dim);
  return 0;
}

extern "C" int cpi_qkv_post(const void* qkv, long qkv_stride, void* q_out, void* k_cache, void* v_cache,
                            int dtype, const int* page_table, int max_blocks, int page_size,
                            const int* token_seq, const int* token_pos, const int* seq_slot,
                            const float* inv_freq, int interleaved, int qk_norm, int norm_before_rope,
                            float norm_eps, int temperature, float floor_scale, float attn_scale,
                            int n_tokens, int n_heads, int n_kv_heads, int head_dim, int write_kv,
                            cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (check_head("qkv_post", n_heads, n_kv_heads, head_dim)) return 1;
  QkvPostParams p{qkv, qkv_stride, q_out, k_cache, v_cache, page_table, max_blocks, page_size,
                  token_seq, token_pos, seq_slot, inv_freq, interleaved, qk_norm, norm_before_rope,
                  norm_eps, temperature, floor_scale, attn_scale, n_heads, n_kv_heads, head_dim, write_kv};
  const int heads_total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (dtype == kBF16 && head_dim == 128 && !interleaved && qkv_stride % 8 == 0 && aligned16(qkv) && aligned16(q_out) &&
      (!write_kv || (aligned16(k_cache) && aligned16(v_cache))) && n_tokens <= 65535) {
    // enough blocks for two waves of the GPU, at most one block per 16 heads
    int slices = (2 * sm_count() * 8 + n_tokens - 1) / n_tokens;
    const int max_slices = (heads_total + 15) / 16;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1) slices = 1;
    int per = (heads_total + slices - 1) / slices;
    per = (per + 1) & ~1;                                        // warps take heads two at a time
    dim3 grid_v(n_tokens, (heads_total + per - 1) / per);
    cpi::launch_pdl(qkv_post_d128_kernel, grid_v, 256, 0, stream, p, per);
    return check_launch("qkv_post");
  }
  dim3 grid(n_tokens, (heads_total + 3) / 4);
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(qkv_post_kernel<T>, grid, 128, 0, stream, p));
  return check_launch("qkv_post");
}

extern "C" int cpi_qkv_prepare(const void* qkv, int in_dtype, long qkv_stride, const void* bias, int bias_dtype,
                               const void* q_norm, const void* k_norm, int norm_dtype, int norm_whole, float norm_eps,
                               const float* inv_freq, int rot_dims, void* q_out, void* k_cache, void* v_cache,
                               int out_dtype, const int* page_table, int max_blocks, int page_size,
                               const int* token_seq, const int* token_pos, const int* seq_slot, int n_tokens,
                               int n_heads, int n_kv_heads, int head_dim, int v_dim, int write_kv, int head_norm,
                               int interleaved, float* v_first, long v_first_stride, const void* v_mix,
                               int v_mix_dtype, int v_mix_mode, int maps, void* q2_out, void* k2_cache, int v_from_k,
                               int temperature, float floor_scale, float attn_scale, float rot_amp,
                               cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
              "qkv_prepare: %d heads cannot be grouped over %d key/value heads", n_heads, n_kv_heads);
  CPI_REQUIRE(head_dim >= 1 && v_dim >= 1, "qkv_prepare: bad head sizes %d / %d", head_dim, v_dim);
  CPI_REQUIRE(inv_freq == nullptr || (rot_dims >= 2 && rot_dims % 2 == 0 && rot_dims <= head_dim),
              "qkv_prepare: %d rotated elements of a head of %d (an even number up to the head size)", rot_dims, head_dim);
  QkvPrepParams p{qkv, qkv_stride, bias, bias_dtype, q_norm, k_norm, norm_dtype, norm_whole, norm_eps, inv_freq,
                  rot_dims, q_out, k_cache, v_cache, page_table, max_blocks, page_size, token_seq, token_pos,
                  seq_slot, n_heads, n_kv_heads, head_dim, v_dim, write_kv, head_norm, interleaved, v_first,
                  v_first_stride, v_mix, v_mix_dtype, v_mix_mode, maps, q2_out, k2_cache, v_from_k, temperature,
                  floor_scale, attn_scale, rot_amp};
  CPI_REQUIRE(maps == 1 || (maps == 2 && q2_out != nullptr && (!write_kv || k2_cache != nullptr)),
              "qkv_prepare: one score map, or two with buffers for the second map's queries and keys");
  CPI_REQUIRE(!v_from_k || (maps == 1 && v_dim == head_dim && v_mix_mode == 0),
              "qkv_prepare: values that are the projected keys have the keys' size, one map and no value mixing");
  CPI_REQUIRE(!temperature || floor_scale > 0.f, "qkv_prepare: a query temperature needs a positive period");
  CPI_REQUIRE(!(head_norm && norm_whole), "qkv_prepare: a norm over the whole projection or one per head, not both");
  CPI_REQUIRE(head_norm >= 0 && head_norm <= 2, "qkv_prepare: unknown kind of head norm %d", head_norm);
  CPI_REQUIRE(v_mix_mode == 0 || (v_first != nullptr && write_kv && (v_mix_mode == 1 || (v_mix_mode == 2 && v_mix))),
              "qkv_prepare: value mixing needs the buffer of the first values (and, to mix, the mixing weight)");
  const size_t row = (size_t)maps * (n_heads + (write_kv ? n_kv_heads : 0)) * head_dim;
  const size_t n_norms = (size_t)maps * (n_heads + n_kv_heads);
  const size_t smem = (head_norm == 1 ? 2 * row + n_norms : head_norm == 2 ? row + n_norms : row) * sizeof(float);
  CPI_REQUIRE(smem <= 200 * 1024, "qkv_prepare: a q and k row of %zu bytes does not fit in shared memory", smem);
  // with few tokens a row is cut along its heads into slices, enough blocks for two per SM (a norm over the whole
  // projection keeps a row in one block, which is then large); a prompt has blocks enough
  const int heads_all = maps * (n_heads + (write_kv ? n_kv_heads : 0));
  int slices = 1;
  if (!norm_whole && n_tokens < 2 * sm_count()) {
    slices = (2 * sm_count() + n_tokens - 1) / n_tokens;
    if (slices > (heads_all + 1) / 2) slices = (heads_all + 1) / 2;
    if (slices < 1) slices = 1;
  }
  const int threads = slices == 1 && n_tokens <= 2 * sm_count() ? 1024 : 256;
#define CPI_PREP(TI, TO)                                                                                       \
  do {                                                                                                         \
    auto kern = qkv_prepare_kernel<TI, TO>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    cpi::launch_pdl(kern, dim3(n_tokens, slices), dim3(threads), smem, stream, p);                                       \
  } while (0)
  if (in_dtype == kF32 && out_dtype == kF32) CPI_PREP(float, float);
  else if (in_dtype == kF32 && out_dtype == kBF16) CPI_PREP(float, __nv_bfloat16);
  else if (in_dtype == kBF16 && out_dtype == kBF16) CPI_PREP(__nv_bfloat16, __nv_bfloat16);
  else { set_error("qkv_prepare: input dtype %d with cache dtype %d is not supported", in_dtype, out_dtype); return 1; }
#undef CPI_PREP
  return check_launch("qkv_prepare");
}

extern "C" int cpi_attention_general(const void* q, void* out, const void* k_cache, const void* v_cache,
                                     int dtype, const int* page_table, int max_blocks, int page_size,
                                     const int* token_seq, const int* token_pos, const int* seq_slot,
                                     int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     int window_kind, int window_size, float scale, const float* score_bias,
                                     int n_dist, const float* sink, int v_dim, int keep_first, float softcap,
                                     cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
              "attention: %d heads cannot be grouped over %d key/value heads", n_heads, n_kv_heads);
  CPI_REQUIRE(head_dim >= 1 && head_dim <= ATT_MAX_DIM && v_dim >= 1 && v_dim <= ATT_MAX_DIM,
              "attention: head sizes %d (keys) and %d (values) are not supported (1 to %d)", head_dim, v_dim, ATT_MAX_DIM);
  CPI_REQUIRE(score_bias == nullptr || n_dist > 0, "attention: a score bias table needs at least one distance");
  CPI_REQUIRE(window_kind == 0 || window_size > 0, "attention: window kind %d needs a size > 0", window_kind);
  CPI_REQUIRE(n_heads <= 65535, "attention: too many heads (%d)", n_heads);
  AttnParams p{q, out, k_cache, v_cache, page_table, max_blocks, page_size, token_seq, token_pos, seq_slot,
               n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, score_bias, n_dist, sink, v_dim,
               window_kind == 2 && keep_first > 0 ? keep_first : 0, softcap};
  dim3 grid(n_tokens, n_heads);
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(attention_general_kernel<T>, grid, ATT_NT, 0, stream, p));
  return check_launch("attention_general");
}
