// Row-wise kernels: token embedding, RMS norm, row gather, expert-output combine.
//
// Formulas (file:line of kurulav1/cpi):
//   embedding   x = Emb[token]                                   src/engine/llama4_cpu_engine.cpp:294-298
//   rmsnorm     y = x * rsqrt(mean(x^2) + eps) * w, fp32 sums    src/engine/llama4_cpu_engine.cpp:47-62,
//                                                                src/kernels/kernels.cu:36-99
// The residual stream is float32 in both precisions; norm outputs take the activation dtype.
#include "common.cuh"

namespace cpi {

template <typename TT>
__global__ void embedding_kernel(const int* __restrict__ tokens, const TT* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {              // never read out of range: flag it and write zeros
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
    return;
  }
  const TT* row = table + (size_t)tok * hidden;
  float* dst = out + (size_t)t * hidden;
  if (sizeof(TT) == 2 && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    // eight elements per thread and load: a row is only a few kilobytes, what counts is one round trip
    const uint4* r16 = reinterpret_cast<const uint4*>(row);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
      const uint4 raw = r16[i];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]), c = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
      reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
      reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

// One block per row.  The sum of squares is taken in a fixed order (thread-strided, then a warp
// tree, then warps in order), so a row's result does not depend on the other rows of the launch.
// Rows of up to 16 elements per thread stay in registers between the two passes.
template <typename TX, typename TO>
__global__ void rmsnorm_kernel(const TX* __restrict__ x, long x_stride, const int* __restrict__ rows,
                               const void* __restrict__ w, int w_dtype, TO* __restrict__ out,
                               long out_stride, int n, float eps, float w_offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const TX* xr = x + (size_t)(rows ? rows[r] : r) * x_stride;
  TO* o = out + (size_t)r * out_stride;
  constexpr int PER = 16;
  if (n <= PER * (int)blockDim.x) {
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = i < n ? to_f32(xr[i]) : 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n) {
        float y = v[j] * inv;
        if (w) y *= w_offset + load_any(w, w_dtype, i);
        o[i] = from_f32<TO>(y);
      }
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_f32(xr[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = to_f32(xr[i]) * inv;
    if (w) v *= w_offset + load_any(w, w_dtype, i);
    o[i] = from_f32<TO>(v);
  }
}

// float32 rows whose length is a multiple of 4: 16-byte loads, the row kept in registers (up to 8192
// elements).  The norm weights are no kernel's output, so they are fetched (as vectors too) before the wait
// on the preceding kernel; after the reduction there is only arithmetic and one vector store per group.
template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_vec4_kernel(const float* __restrict__ x, long x_stride,
                                                           const int* __restrict__ rows, const void* __restrict__ w,
                                                           int w_dtype, TO* __restrict__ out, long out_stride, int n,
                                                           float eps, float w_offset) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  constexpr int PER = 8;
  const int r = blockIdx.x, n4 = n >> 2;
  float4 g[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    g[j] = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w && i < n4) {
      if (w_dtype == kF32) {
        g[j] = reinterpret_cast<const float4*>(w)[i];
      } else {
        const uint2 raw = reinterpret_cast<const uint2*>(w)[i];
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        g[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
      g[j].x += w_offset; g[j].y += w_offset; g[j].z += w_offset; g[j].w += w_offset;
    }
  }
  pdl_wait();
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * x_stride);
  float4 v[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    v[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  TO* o = out + (size_t)r * out_stride;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n4) {
      // (x * inv) * weight, in this order, as the scalar kernel does
      const float y0 = v[j].x * inv * g[j].x, y1 = v[j].y * inv * g[j].y, y2 = v[j].z * inv * g[j].z, y3 = v[j].w * inv * g[j].w;
      if (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + 4 * i) = make_float4(y0, y1, y2, y3);
      } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(o) + 4 * i) = pk;
      }
    }
  }
}

// residual[t] += sum_k y[row_of_slot[t*K + k]] in the order k = 0..K-1.
template <typename TY>
__global__ void moe_combine_kernel(float* __restrict__ residual, const TY* __restrict__ y,
                                   const int* __restrict__ row_of_slot, int top_k, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
    float acc = residual[(size_t)t * hidden + i];
    for (int k = 0; k < top_k; ++k) {
      const int r = row_of_slot[t * top_k + k];
      acc += to_f32(y[(size_t)r * hidden + i]);
    }
    residual[(size_t)t * hidden + i] = acc;
  }
}

__device__ __forceinline__ float4 load4_f32(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_f32(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// The same sum, four features per thread and one pass: every load of a thread is in flight at once
// (hidden a multiple of 4, all rows 16-byte aligned).  Same order of additions, so the same bits.
template <typename TY>
__global__ void moe_combine_vec4_kernel(float* __restrict__ residual, const TY* __restrict__ y,
                                        const int* __restrict__ row_of_slot, int top_k, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (i >= hidden) return;
  float* res = residual + (size_t)t * hidden + i;
  float4 acc = load4_f32(res);
  for (int k0 = 0; k0 < top_k; k0 += 4) {
    float4 v[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      if (k0 + kk < top_k) v[kk] = load4_f32(y + (size_t)row_of_slot[t * top_k + k0 + kk] * hidden + i);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      if (k0 + kk < top_k) { acc.x += v[kk].x; acc.y += v[kk].y; acc.z += v[kk].z; acc.w += v[kk].w; }
  }
  *reinterpret_cast<float4*>(res) = acc;
}

// act(gate) * up over rows [gate | up]; act: 0 silu, 1 the tanh form of gelu
// 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
__device__ __forceinline__ float gate_act(float a, int act) {
  if (act == 1) return 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
  return a / (1.0f + expf(-a));
}

// act 2, the clamped form: g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float clamped_gate_mul(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

template <typename TI, typename T>
__global__ void swiglu_kernel(const TI* __restrict__ gu, T* __restrict__ out, int inter, int act, float limit) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const TI* g = gu + (size_t)t * 2 * inter;
  for (int i = threadIdx.x; i < inter; i += blockDim.x) {
    const float a = to_f32(g[i]), b = to_f32(g[inter + i]);
    out[(size_t)t * inter + i] = from_f32<T>(act == 2 ? clamped_gate_mul(a, b, limit) : gate_act(a, act) * b);
  }
}

// Branches that are normalised before they are summed: out[t] (+)= scale * sum_b rmsnorm(y_b[t]) * w_b, each branch
// by its own mean square over the row (float32 rows in, float32 out; weights of any dtype).
constexpr int kMaxBranches = 4;
struct BranchSumParams {
  const float* y[kMaxBranches]; long y_stride[kMaxBranches]; const void* w[kMaxBranches];
  int w_dtype, n_branches, width, add;
  float eps, scale;
  float* out; long out_stride;
};

__global__ void __launch_bounds__(256) branch_norm_sum_kernel(BranchSumParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float inv[kMaxBranches];
#pragma unroll
  for (int b = 0; b < kMaxBranches; ++b) {
    inv[b] = 0.f;
    if (b < p.n_branches) {
      const float* y = p.y[b] + (size_t)t * p.y_stride[b];
      float ss = 0.f;
      for (int i = threadIdx.x; i < p.width; i += blockDim.x) ss = fmaf(y[i], y[i], ss);
      inv[b] = 1.0f / sqrtf(block_sum(ss, scratch) / (float)p.width + p.eps);
    }
  }
  float* o = p.out + (size_t)t * p.out_stride;
  for (int i = threadIdx.x; i < p.width; i += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < kMaxBranches; ++b)
      if (b < p.n_branches) acc += p.y[b][(size_t)t * p.y_stride[b] + i] * inv[b] * load_any(p.w[b], p.w_dtype, i);
    acc *= p.scale;
    o[i] = p.add ? o[i] + acc : acc;
  }
}

// A sublayer's output enters the residual through a norm of its own:
//   out[t] (+)= rmsnorm(sum_b scale_b * y_b[t]) * w,     and optionally   h_out[t] = out[t] in another dtype
// (the sublayer's output may be several branches with a constant each; h_out is the next sublayer's input when the
// sublayers read the residual itself).  One block per token, float32 throughout.
struct SumNormAddParams {
  const float* y[kMaxBranches]; long y_stride[kMaxBranches]; float scale[kMaxBranches];
  const void* w; int w_dtype; int n_branches, width, add; float eps;
  float* out; long out_stride;
  void* h_out; long h_stride;
  int normalise;                         // 0: the scaled sum enters as it is
};

template <typename TH>
__global__ void __launch_bounds__(256) sum_norm_add_kernel(SumNormAddParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  auto branches = [&](int i) {
    float v = 0.f;
#pragma unroll
    for (int b = 0; b < kMaxBranches; ++b)
      if (b < p.n_branches) v = fmaf(p.scale[b], p.y[b][(size_t)t * p.y_stride[b] + i], v);
    return v;
  };
  float inv = 1.0f;
  if (p.normalise) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.width; i += blockDim.x) { const float v = branches(i); ss = fmaf(v, v, ss); }
    inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)p.width + p.eps);
  }
  float* o = p.out + (size_t)t * p.out_stride;
  TH* h = p.h_out ? reinterpret_cast<TH*>(p.h_out) + (size_t)t * p.h_stride : nullptr;
  for (int i = threadIdx.x; i < p.width; i += blockDim.x) {
    float v = branches(i) * inv;
    if (p.w) v *= load_any(p.w, p.w_dtype, i);
    if (p.add) v += o[i];
    o[i] = v;
    if (h) h[i] = from_f32<TH>(v);
  }
}

// The same for rows of up to 8,192 elements that are multiples of four and start on 16-byte boundaries: a thread keeps
// its (up to eight) groups of four sums in registers between the two passes and moves 16 bytes at a time.  Same
// sums in the same order per element; the row's sum of squares is taken in another order.
template <typename TH>
__global__ void __launch_bounds__(256) sum_norm_add_vec_kernel(SumNormAddParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x, groups = p.width >> 2;
  float4 v[8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = threadIdx.x + j * 256;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (g < groups) {
#pragma unroll
      for (int b = 0; b < kMaxBranches; ++b)
        if (b < p.n_branches) {
          const float4 y = *reinterpret_cast<const float4*>(p.y[b] + (size_t)t * p.y_stride[b] + 4 * g);
          v[j].x = fmaf(p.scale[b], y.x, v[j].x); v[j].y = fmaf(p.scale[b], y.y, v[j].y);
          v[j].z = fmaf(p.scale[b], y.z, v[j].z); v[j].w = fmaf(p.scale[b], y.w, v[j].w);
        }
      ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
    }
  }
  const float inv = p.normalise ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)p.width + p.eps) : 1.0f;
  float* o = p.out + (size_t)t * p.out_stride;
  TH* h = p.h_out ? reinterpret_cast<TH*>(p.h_out) + (size_t)t * p.h_stride : nullptr;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = threadIdx.x + j * 256;
    if (g >= groups) continue;
    float r[4] = {v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv};
    if (p.w) {
#pragma unroll
      for (int e = 0; e < 4; ++e) r[e] *= load_any(p.w, p.w_dtype, 4 * g + e);
    }
    if (p.add) {
      const float4 old = *reinterpret_cast<const float4*>(o + 4 * g);
      r[0] += old.x; r[1] += old.y; r[2] += old.z; r[3] += old.w;
    }
    *reinterpret_cast<float4*>(o + 4 * g) = make_float4(r[0], r[1], r[2], r[3]);
    if (h) {
#pragma unroll
      for (int e = 0; e < 4; ++e) h[4 * g + e] = from_f32<TH>(r[e]);
    }
  }
}

// out[t, :] (+)= bias: float32 rows that a product then adds into, so that the product carries a bias
__global__ void __launch_bounds__(256) bias_rows_kernel(float* __restrict__ out, long out_stride, const void* bias,
                                                        int bias_dtype, int width, int add) {
  pdl_launch_dependents();
  pdl_wait();
  float* o = out + (size_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float b = load_any(bias, bias_dtype, i);
    o[i] = add ? o[i] + b : b;
  }
}

// out[t] = [a[t] | b[t]] in out's dtype: two float32 rows side by side as one operand row of a product
template <typename TO>
__global__ void __launch_bounds__(256) concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          TO* __restrict__ out, int wa, int wb) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  TO* o = out + (size_t)t * (wa + wb);
  for (int i = threadIdx.x; i < wa + wb; i += blockDim.x)
    o[i] = from_f32<TO>(i < wa ? a[(size_t)t * wa + i] : b[(size_t)t * wb + i - wa]);
}

// logits <- cap * tanh(logits * scale / cap), or logits * scale when cap is 0.
__global__ void logit_post_kernel(float* __restrict__ logits, long n, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float v = logits[i] * scale;
    logits[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

// dst[r, :] = src[rows[r], :]  (16-byte chunks; width * sizeof(T) must be a multiple of 16)
__global__ void gather_rows_kernel(const uint4* __restrict__ src, long src_stride16, const int* __restrict__ rows,
                                   uint4* __restrict__ dst, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const uint4* s = src + (size_t)rows[r] * src_stride16;
  uint4* d = dst + (size_t)r * chunks;
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) d[i] = s[i];
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_gather_rows(const void* src, long src_stride_bytes, const int* rows, void* dst, int n_rows,
                               int row_bytes, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(row_bytes % 16 == 0 && src_stride_bytes % 16 == 0, "gather_rows: rows of %d bytes (stride %ld) are not 16-byte multiples", row_bytes, src_stride_bytes);
  cpi::launch_pdl(gather_rows_kernel, n_rows, 128, 0, stream, (const uint4*)src, src_stride_bytes / 16, rows, (uint4*)dst, row_bytes / 16);
  return check_launch("gather_rows");
}

extern "C" int cpi_embedding(const int* tokens, const void* table, int table_dtype, float* out,
                             int n_tokens, int hidden, int vocab, int* err_flag, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d", n_tokens, hidden, vocab);
  CPI_DISPATCH_DTYPE(table_dtype, TT,
      cpi::launch_pdl(embedding_kernel<TT>, n_tokens, 256, 0, stream, tokens, (const TT*)table, out, hidden, vocab, err_flag));
  return check_launch("embedding");
}

extern "C" int cpi_rmsnorm(const void* x, int x_dtype, long x_stride, const int* rows, const void* w,
                           int w_dtype, void* out, int out_dtype, long out_stride, int n_rows, int n,
                           float eps, float w_offset, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(n_rows > 0 && n > 0, "rmsnorm: bad sizes rows=%d n=%d", n_rows, n);
  const int out_esz = out_dtype == kF32 ? 4 : 2;
  if (x_dtype == kF32 && n % 4 == 0 && n >= 1024 && n <= 8192 && x_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (out_stride * out_esz) % 16 == 0) {
    CPI_DISPATCH_DTYPE(out_dtype, TO,
        (cpi::launch_pdl(rmsnorm_vec4_kernel<TO>, n_rows, 256, 0, stream, (const float*)x, x_stride, rows, w, w_dtype,
                         (TO*)out, out_stride, n, eps, w_offset)));
    return check_launch("rmsnorm");
  }
  const int threads = n <= 256 ? 64 : (n <= 2048 ? 256 : 512);
  CPI_DISPATCH_DTYPE(x_dtype, TX, CPI_DISPATCH_DTYPE(out_dtype, TO,
      (cpi::launch_pdl(rmsnorm_kernel<TX, TO>, n_rows, threads, 0, stream, (const TX*)x, x_stride, rows, w, w_dtype,
                                                              (TO*)out, out_stride, n, eps, w_offset))));
  return check_launch("rmsnorm");
}

extern "C" int cpi_moe_combine(float* residual, const void* y, int y_dtype, const int* row_of_slot,
                               int n_tokens, int top_k, int hidden, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  const bool vec = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (y_dtype == kF32 || y_dtype == kBF16);
  if (vec) {
    const dim3 grid(n_tokens, (hidden / 4 + 127) / 128);
    if (y_dtype == kF32)
      cpi::launch_pdl(moe_combine_vec4_kernel<float>, grid, 128, 0, stream, residual, (const float*)y, row_of_slot, top_k, hidden);
    else
      cpi::launch_pdl(moe_combine_vec4_kernel<__nv_bfloat16>, grid, 128, 0, stream, residual, (const __nv_bfloat16*)y, row_of_slot, top_k, hidden);
    return check_launch("moe_combine");
  }
  CPI_DISPATCH_DTYPE(y_dtype, TY,
      cpi::launch_pdl(moe_combine_kernel<TY>, dim3(n_tokens, 1), 256, 0, stream, residual, (const TY*)y, row_of_slot, top_k, hidden));
  return check_launch("moe_combine");
}

extern "C" int cpi_swiglu(const void* gate_up, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(swiglu_kernel<T, T>, n_rows, 256, 0, stream, (const T*)gate_up, (T*)out, inter, 0, 0.f));
  return check_launch("swiglu");
}

// out = act(gate) * up for rows [gate | up] of float32 or of out's dtype; act 0 = silu, 1 = gelu (tanh form),
// 2 = the clamped form min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)
extern "C" int cpi_gated_act(const void* gate_up, int in_dtype, void* out, int out_dtype, int n_rows, int inter,
                             int act, float limit, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(act >= 0 && act <= 2, "gated_act: unknown activation %d", act);
  if (in_dtype == kF32) {
    CPI_DISPATCH_DTYPE(out_dtype, T, cpi::launch_pdl(swiglu_kernel<float, T>, n_rows, 256, 0, stream, (const float*)gate_up, (T*)out, inter, act, limit));
  } else {
    CPI_REQUIRE(in_dtype == out_dtype, "gated_act: bfloat16 rows give bfloat16 rows");
    cpi::launch_pdl(swiglu_kernel<__nv_bfloat16, __nv_bfloat16>, n_rows, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, act, limit);
  }
  return check_launch("gated_act");
}

extern "C" int cpi_logit_post(float* logits, long n, float scale, float cap, cudaStream_t stream) {
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  cpi::launch_pdl(logit_post_kernel, blocks, 256, 0, stream, logits, n, scale, cap);
  return check_launch("logit_post");
}

extern "C" int cpi_branch_norm_sum(const float* const* y, const long* y_stride, const void* const* w, int w_dtype,
                                   int n_branches, int n_rows, int width, float eps, float scale, int add, float* out,
                                   long out_stride, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(n_branches >= 1 && n_branches <= kMaxBranches, "branch_norm_sum: %d branches (1 to %d)", n_branches, kMaxBranches);
  BranchSumParams p{};
  for (int b = 0; b < n_branches; ++b) { p.y[b] = y[b]; p.y_stride[b] = y_stride[b]; p.w[b] = w[b]; }
  p.w_dtype = w_dtype; p.n_branches = n_branches; p.width = width; p.add = add; p.eps = eps; p.scale = scale;
  p.out = out; p.out_stride = out_stride;
  cpi::launch_pdl(branch_norm_sum_kernel, n_rows, 256, 0, stream, p);
  return check_launch("branch_norm_sum");
}

extern "C" int cpi_sum_norm_add(const float* const* y, const long* y_stride, const float* scale, int n_branches,
                                const void* w, int w_dtype, int n_rows, int width, float eps, int add, float* out,
                                long out_stride, void* h_out, int h_dtype, long h_stride, int normalise,
                                cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(n_branches >= 1 && n_branches <= kMaxBranches, "sum_norm_add: %d branches (1 to %d)", n_branches, kMaxBranches);
  SumNormAddParams p{};
  for (int b = 0; b < n_branches; ++b) { p.y[b] = y[b]; p.y_stride[b] = y_stride[b]; p.scale[b] = scale[b]; }
  p.w = w; p.w_dtype = w_dtype; p.n_branches = n_branches; p.width = width; p.add = add; p.eps = eps;
  p.out = out; p.out_stride = out_stride; p.h_out = h_out; p.h_stride = h_stride; p.normalise = normalise;
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  bool vec = width % 4 == 0 && width <= 8192 && aligned16(out) && out_stride % 4 == 0;
  for (int b = 0; b < n_branches; ++b) vec = vec && aligned16(y[b]) && y_stride[b] % 4 == 0;
  if (vec) CPI_DISPATCH_DTYPE(h_dtype, TH, cpi::launch_pdl(sum_norm_add_vec_kernel<TH>, n_rows, 256, 0, stream, p));
  else CPI_DISPATCH_DTYPE(h_dtype, TH, cpi::launch_pdl(sum_norm_add_kernel<TH>, n_rows, 256, 0, stream, p));
  return check_launch("sum_norm_add");
}

extern "C" int cpi_bias_rows(float* out, long out_stride, const void* bias, int bias_dtype, int n_rows, int width,
                             int add, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  cpi::launch_pdl(bias_rows_kernel, n_rows, 256, 0, stream, out, out_stride, bias, bias_dtype, width, add);
  return check_launch("bias_rows");
}

extern "C" int cpi_concat_rows(const float* a, const float* b, void* out, int out_dtype, int n_rows, int wa, int wb,
                               cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_DISPATCH_DTYPE(out_dtype, TO, cpi::launch_pdl(concat_rows_kernel<TO>, n_rows, 256, 0, stream, a, b, (TO*)out, wa, wb));
  return check_launch("concat_rows");
}
