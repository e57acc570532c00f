// Row kernels of attention over a cached latent, and of a gated per-token side input.
//
// Latent attention keeps, per position, one vector c (an RMS-normed low-rank projection of the layer's input) and one
// rotated key part r that all heads share; a head's key is [W_uk,h c | r] and its value W_uv,h c.  Because a score
// q_h . W_uk,h c equals (W_uk,h^T q_h) . c, attention runs over the cached rows [c | r] themselves, as one key/value
// head that every query head reads: the query is [W_uk,h^T q_h | rotated part], the output a weighted sum of rows
// [c | r] whose first part then goes through W_uv,h.  The two per-head products are grouped matrix products with one
// group per head, over rows laid out head by head ("head-major": row h * T + t), which these kernels produce.
//
//   latent_kv_write     per token: c = rmsnorm(x[:rank]) * w, r = rotate(x[rank:rank + R]); the row [c | r] goes into
//                       the cache page of the token's position (one head of rank + R elements).
//   latent_q_split      per token and head, from q [T, H, D + R] (float32): the first D elements go to the head-major
//                       rows plain[h * T + t, :D]; the last R, rotated, to full[t, h, rank:rank + R].  Also fills the
//                       lists a grouped product over heads needs: offsets[h] = h * T and rows[h * T + t] = t * H + h.
//   head_major_rows     out[h * T + t, :n] = in[t, h, :n] for rows in[t, h, :] of `in_dim` elements.
//   gated_side_input    x[t] += rmsnorm(P (gelu_tanh(G x[t]) * e[t])) * w with e[t] = table[token[t], off : off + n]:
//                       a small per-token vector looked up by token id, gated by a projection of the residual,
//                       projected up to the model width, normed and added.  Everything in float32.
//   cast_rows, side_gate_act   the pieces of the same around two products on the tensor cores (bfloat16 operands).
#include "common.cuh"

namespace cpi {

__device__ __forceinline__ void pair_of(int d, int half, int interleaved, bool& first, int& other, int& f) {
  if (interleaved) { first = !(d & 1); other = d ^ 1; f = d >> 1; }
  else { first = d < half; other = first ? d + half : d - half; f = first ? d : d - half; }
}

struct LatentKvParams {
  const float* x; long x_stride;                 // [T, rank + R]
  const void* norm_w; int norm_dtype; float eps; // [rank] or null
  const float* inv_freq; int interleaved;        // [R / 2] or null
  void* cache;                                   // [pages, 1, page_size, rank + R]
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  int rank, rot;
};

template <typename TO>
__global__ void __launch_bounds__(256) latent_kv_write_kernel(LatentKvParams p) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* x = p.x + (size_t)t * p.x_stride;
  const int pos = p.token_pos[t];
  const int slot = p.seq_slot[p.token_seq[t]];
  const int page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
  const int W = p.rank + p.rot;
  TO* dst = reinterpret_cast<TO*>(p.cache) + ((size_t)page * p.page_size + pos % p.page_size) * W;
  float ss = 0.f;
  for (int i = tid; i < p.rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
  for (int i = tid; i < p.rank; i += blockDim.x) {
    float v = x[i] * inv;
    if (p.norm_w) v *= load_any(p.norm_w, p.norm_dtype, i);
    dst[i] = from_f32<TO>(v);
  }
  const int half = p.rot >> 1;
  for (int d = tid; d < p.rot; d += blockDim.x) {
    float v = x[p.rank + d];
    if (p.inv_freq) {
      bool first; int od, f;
      pair_of(d, half, p.interleaved, first, od, f);
      const float other = x[p.rank + od];
      float sn, cs;
      sincosf((float)pos * p.inv_freq[f], &sn, &cs);
      v = first ? v * cs - other * sn : v * cs + other * sn;
    }
    dst[p.rank + d] = from_f32<TO>(v);
  }
}

struct LatentQParams {
  const float* q; long q_stride;                 // [T, H (D + R)]
  const float* inv_freq; int interleaved;
  void* plain;                                   // [H T, D] head-major
  void* full;                                    // [T, H, rank + R]
  int* offsets; int* rows;                       // [H + 1], [H T]
  const int* token_pos;
  int n_tokens, n_heads, dim, rot, rank;
};

template <typename TO>
__global__ void __launch_bounds__(256) latent_q_split_kernel(LatentQParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = p.n_heads, D = p.dim, R = p.rot, T = p.n_tokens;
  const float* q = p.q + (size_t)t * p.q_stride;
  const int pos = p.token_pos[t];
  const int half = R >> 1, W = p.rank + R;
  TO* plain = reinterpret_cast<TO*>(p.plain);
  TO* full = reinterpret_cast<TO*>(p.full) + (size_t)t * H * W;
  for (int i = tid; i < H * (D + R); i += blockDim.x) {
    const int h = i / (D + R), d = i % (D + R);
    float v = q[i];
    if (d < D) {
      plain[((size_t)h * T + t) * D + d] = from_f32<TO>(v);
    } else {
      const int r = d - D;
      if (p.inv_freq) {
        bool first; int od, f;
        pair_of(r, half, p.interleaved, first, od, f);
        const float other = q[i - r + od];
        float sn, cs;
        sincosf((float)pos * p.inv_freq[f], &sn, &cs);
        v = first ? v * cs - other * sn : v * cs + other * sn;
      }
      full[(size_t)h * W + p.rank + r] = from_f32<TO>(v);
    }
  }
  for (int h = tid; h < H; h += blockDim.x) p.rows[(size_t)h * T + t] = t * H + h;
  if (t == 0)
    for (int h = tid; h <= H; h += blockDim.x) p.offsets[h] = h * T;
}

template <typename TO>
__global__ void __launch_bounds__(256) head_major_rows_kernel(const TO* in, TO* out, int n_tokens, int n_heads,
                                                              int in_dim, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const TO* src = in + (size_t)t * n_heads * in_dim;
  for (int i = threadIdx.x; i < n_heads * n; i += blockDim.x) {
    const int h = i / n, d = i % n;
    out[((size_t)h * n_tokens + t) * n + d] = src[(size_t)h * in_dim + d];
  }
}

// ---- the gated side input ---------------------------------------------------------------------------------
struct SideParams {
  float* x; long x_stride;                       // residual [T, W], updated in place
  const int* tokens;
  const void* table; int table_dtype; long table_stride; int table_offset; int vocab;      // [vocab, *]
  const void* gate; const void* proj; int w_dtype;       // [n, W], [W, n]
  const void* norm_w; int norm_dtype; float eps;         // [W]
  int width, n, n_tokens;
};

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A block takes TPB consecutive tokens, so that a weight element read once serves all of them.  The order of every
// sum of a token is the same for every TPB and every place in the block: a row does not depend on its neighbours.
template <typename TW, int TPB>
__global__ void __launch_bounds__(256) gated_side_input_kernel(SideParams p) {
  pdl_launch_dependents();
  extern __shared__ float sm[];                  // x rows [TPB][W], g [TPB][n]
  __shared__ float scratch[32];
  pdl_wait();
  const int t0 = blockIdx.x * TPB, tid = threadIdx.x, W = p.width, n = p.n;
  const int nt = min(TPB, p.n_tokens - t0);
  float* xs = sm;
  float* g = sm + (size_t)TPB * W;
  const TW* gate = reinterpret_cast<const TW*>(p.gate);
  const TW* proj = reinterpret_cast<const TW*>(p.proj);
  for (int k = 0; k < TPB; ++k) {
    const float* x = p.x + (size_t)(t0 + min(k, nt - 1)) * p.x_stride;
    for (int i = tid; i < W; i += blockDim.x) xs[(size_t)k * W + i] = x[i];
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  for (int j = warp; j < n; j += nw) {
    float dot[TPB];
#pragma unroll
    for (int k = 0; k < TPB; ++k) dot[k] = 0.f;
    const TW* gr = gate + (size_t)j * W;
    for (int i = lane; i < W; i += 32) {
      const float w = to_f32(gr[i]);
#pragma unroll
      for (int k = 0; k < TPB; ++k) dot[k] = fmaf(w, xs[(size_t)k * W + i], dot[k]);
    }
#pragma unroll
    for (int k = 0; k < TPB; ++k) {
      const float d = warp_sum(dot[k]);
      if (lane == 0 && k < nt) {
        int tok = p.tokens[t0 + k];
        tok = min(max(tok, 0), p.vocab - 1);     // the embedding kernel has flagged a token outside the table
        g[k * n + j] = gelu_tanh_f(d) * load_any(p.table, p.table_dtype, (size_t)tok * p.table_stride + p.table_offset + j);
      }
    }
  }
  __syncthreads();
  float ss[TPB];
#pragma unroll
  for (int k = 0; k < TPB; ++k) ss[k] = 0.f;
  for (int c = tid; c < W; c += blockDim.x) {
    float y[TPB];
#pragma unroll
    for (int k = 0; k < TPB; ++k) y[k] = 0.f;
    const TW* pr = proj + (size_t)c * n;
    int j = 0;
    if (sizeof(TW) == 2 && n % 8 == 0) {         // rows of the projection start on 16 bytes: eight weights a load
      for (; j < n; j += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(pr + j);
        const __nv_bfloat16* w8 = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float w = __bfloat162float(w8[u]);
#pragma unroll
          for (int k = 0; k < TPB; ++k) y[k] = fmaf(w, g[k * n + j + u], y[k]);
        }
      }
    }
    for (; j < n; ++j) {
      const float w = to_f32(pr[j]);
#pragma unroll
      for (int k = 0; k < TPB; ++k) y[k] = fmaf(w, g[k * n + j], y[k]);
    }
#pragma unroll
    for (int k = 0; k < TPB; ++k) {
      ss[k] = fmaf(y[k], y[k], ss[k]);
      xs[(size_t)k * W + c] = y[k];              // a thread reads back only what it wrote
    }
  }
#pragma unroll
  for (int k = 0; k < TPB; ++k) {
    const float tot = block_sum(ss[k], scratch);
    if (k >= nt) continue;
    const float inv = 1.0f / sqrtf(tot / (float)W + p.eps);
    float* x = p.x + (size_t)(t0 + k) * p.x_stride;
    for (int c = tid; c < W; c += blockDim.x) {
      float y = xs[(size_t)k * W + c] * inv;
      if (p.norm_w) y *= load_any(p.norm_w, p.norm_dtype, c);
      x[c] += y;
    }
  }
}

// The same in pieces, for the products on the tensor cores: out = x in another dtype, and
// g[t, j] = gelu_tanh(z[t, j]) * table[token[t], off + j] for the float32 result z of the gate product.
template <typename TO>
__global__ void __launch_bounds__(256) cast_rows_kernel(const float* x, long x_stride, TO* out, int n_rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<TO>(x[(i / n) * x_stride + i % n]);
}

template <typename TO>
__global__ void __launch_bounds__(256) side_gate_act_kernel(const float* z, const int* tokens, const void* table,
                                                            int table_dtype, long table_stride, int table_offset,
                                                            int vocab, TO* out, int n_rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / n, j = i % n;
    const int tok = min(max(tokens[t], 0), vocab - 1);
    out[i] = from_f32<TO>(gelu_tanh_f(z[i]) * load_any(table, table_dtype, (size_t)tok * table_stride + table_offset + j));
  }
}

// out = relu(x)^2 over rows (float32 in, any dtype out; in place when the two are one buffer)
template <typename TO>
__global__ void __launch_bounds__(256) relu_squared_kernel(const float* x, long x_stride, TO* out, long out_stride,
                                                           int n_rows, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n, c = i % n;
    const float v = fmaxf(x[r * x_stride + c], 0.f);
    out[r * out_stride + c] = from_f32<TO>(v * v);
  }
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_latent_kv_write(const float* x, long x_stride, const void* norm_w, int norm_dtype, float eps,
                                   const float* inv_freq, int interleaved, void* cache, int cache_dtype,
                                   const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                   const int* token_pos, const int* seq_slot, int n_tokens, int rank, int rot,
                                   cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(rank >= 1 && rot >= 0 && rot % 2 == 0, "latent_kv_write: a latent of %d and a rotated part of %d", rank, rot);
  LatentKvParams p{x, x_stride, norm_w, norm_dtype, eps, inv_freq, interleaved, cache, page_table, max_blocks,
                   page_size, token_seq, token_pos, seq_slot, rank, rot};
  CPI_DISPATCH_DTYPE(cache_dtype, T, cpi::launch_pdl(latent_kv_write_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, p));
  return check_launch("latent_kv_write");
}

extern "C" int cpi_latent_q_split(const float* q, long q_stride, const float* inv_freq, int interleaved, void* plain,
                                  void* full, int out_dtype, int* offsets, int* rows, const int* token_pos,
                                  int n_tokens, int n_heads, int dim, int rot, int rank, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_heads >= 1 && dim >= 1 && rot >= 0 && rot % 2 == 0 && rank >= 1,
              "latent_q_split: bad sizes heads=%d dim=%d rotated=%d rank=%d", n_heads, dim, rot, rank);
  LatentQParams p{q, q_stride, inv_freq, interleaved, plain, full, offsets, rows, token_pos, n_tokens, n_heads, dim,
                  rot, rank};
  CPI_DISPATCH_DTYPE(out_dtype, T, cpi::launch_pdl(latent_q_split_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, p));
  return check_launch("latent_q_split");
}

extern "C" int cpi_head_major_rows(const void* in, void* out, int dtype, int n_tokens, int n_heads, int in_dim, int n,
                                   cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_heads >= 1 && n >= 1 && n <= in_dim, "head_major_rows: %d of %d elements of %d heads", n, in_dim, n_heads);
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(head_major_rows_kernel<T>, dim3(n_tokens), dim3(256), 0, stream,
                                               reinterpret_cast<const T*>(in), reinterpret_cast<T*>(out), n_tokens,
                                               n_heads, in_dim, n));
  return check_launch("head_major_rows");
}

extern "C" int cpi_gated_side_input(float* x, long x_stride, const int* tokens, const void* table, int table_dtype,
                                    long table_stride, int table_offset, int vocab, const void* gate, const void* proj,
                                    int w_dtype, const void* norm_w, int norm_dtype, float eps, int n_tokens, int width,
                                    int n, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(width >= 1 && n >= 1 && vocab >= 1, "gated_side_input: bad sizes width=%d n=%d vocab=%d", width, n, vocab);
  const size_t row = (size_t)(width + n) * sizeof(float);
  CPI_REQUIRE(row <= 200 * 1024, "gated_side_input: a row of %d + %d floats does not fit in shared memory", width, n);
  // tokens a block takes: as many as fit, and no more than leave every multiprocessor a block
  int tpb = 8;
  while (tpb > 1 && (row * tpb > 200 * 1024 || (n_tokens + tpb - 1) / tpb < sm_count())) tpb >>= 1;
  SideParams p{x, x_stride, tokens, table, table_dtype, table_stride, table_offset, vocab, gate, proj, w_dtype,
               norm_w, norm_dtype, eps, width, n, n_tokens};
  const size_t smem = row * tpb;
  const dim3 grid((n_tokens + tpb - 1) / tpb);
#define CPI_SIDE_LAUNCH(TW, TPB)                                                                                  \
  do {                                                                                                            \
    if (smem > 48 * 1024)                                                                                         \
      cudaFuncSetAttribute(gated_side_input_kernel<TW, TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    cpi::launch_pdl(gated_side_input_kernel<TW, TPB>, grid, dim3(256), smem, stream, p);                          \
  } while (0)
  CPI_DISPATCH_DTYPE(w_dtype, TW, {
    if (tpb == 8) CPI_SIDE_LAUNCH(TW, 8);
    else if (tpb == 4) CPI_SIDE_LAUNCH(TW, 4);
    else if (tpb == 2) CPI_SIDE_LAUNCH(TW, 2);
    else CPI_SIDE_LAUNCH(TW, 1);
  });
#undef CPI_SIDE_LAUNCH
  return check_launch("gated_side_input");
}

static int row_blocks(size_t total) {
  const size_t want = (total + 255) / 256, most = (size_t)8 * sm_count();
  return (int)(want < most ? want : most);
}

extern "C" int cpi_cast_rows(const float* x, long x_stride, void* out, int out_dtype, int n_rows, int n,
                             cudaStream_t stream) {
  if (n_rows == 0 || n == 0) return 0;
  CPI_DISPATCH_DTYPE(out_dtype, T, cpi::launch_pdl(cast_rows_kernel<T>, dim3(row_blocks((size_t)n_rows * n)), dim3(256), 0,
                                                   stream, x, x_stride, reinterpret_cast<T*>(out), n_rows, n));
  return check_launch("cast_rows");
}

extern "C" int cpi_side_gate_act(const float* z, const int* tokens, const void* table, int table_dtype,
                                 long table_stride, int table_offset, int vocab, void* out, int out_dtype, int n_rows,
                                 int n, cudaStream_t stream) {
  if (n_rows == 0 || n == 0) return 0;
  CPI_REQUIRE(vocab >= 1 && table_offset >= 0, "side_gate_act: bad sizes vocab=%d offset=%d", vocab, table_offset);
  CPI_DISPATCH_DTYPE(out_dtype, T, cpi::launch_pdl(side_gate_act_kernel<T>, dim3(row_blocks((size_t)n_rows * n)), dim3(256),
                                                   0, stream, z, tokens, table, table_dtype, table_stride, table_offset,
                                                   vocab, reinterpret_cast<T*>(out), n_rows, n));
  return check_launch("side_gate_act");
}

extern "C" int cpi_relu_squared(const float* x, long x_stride, void* out, int out_dtype, long out_stride, int n_rows,
                                int n, cudaStream_t stream) {
  if (n_rows == 0 || n == 0) return 0;
  const size_t total = (size_t)n_rows * n;
  const int blocks = (int)((total + 255) / 256 < (size_t)(8 * sm_count()) ? (total + 255) / 256 : 8 * sm_count());
  CPI_DISPATCH_DTYPE(out_dtype, T, cpi::launch_pdl(relu_squared_kernel<T>, dim3(blocks), dim3(256), 0, stream, x, x_stride,
                                                   reinterpret_cast<T*>(out), out_stride, n_rows, n));
  return check_launch("relu_squared");
}
