// Softmax attention over cached latent rows, in bfloat16 on the warp-level tensor-core path (mma.sync m16n8k16).
//
// Every position keeps ONE row [c | r] of `row` = rank + rot elements that all query heads share: the row is the key
// (all of it) and the value (its first `rank` elements).  A query row is one (token, head) pair, already taken
// through the key up-projection, so the rows of a block are the heads of a few consecutive tokens of one sequence
// stacked: 64 rows against tiles of 32 cached positions.
//
//   S = Q K^T         8 warps: warp (g, c) owns query rows [16 g, 16 g + 16) and key columns [16 c, 16 c + 16) of
//                     the tile; fragments through ldmatrix from padded shared-memory rows; S * scale * log2(e),
//                     masked by position, goes to shared memory in float32
//   P = 2^(S - m)     each warp for its 16 rows (the two warps of a row group compute the same numbers, after a
//                     barrier of their own): running maximum and sum in float32, P rounded to bfloat16 as the A
//                     operand; the accumulators are rescaled only when a maximum of the warp's rows has grown
//   O += P V          warp (g, c) accumulates rows [16 g, +16) x value columns [c * CH, (c + 1) * CH) in registers
//                     (CH = 8 NT, NT = 8, 16 or 32 by the latent's size); V fragments through ldmatrix.trans
//                     from the same shared-memory tile that held the keys
// Key/value tiles are fetched with cp.async into two buffers, tile i + 1 while tile i is computed.  Rows of a tile
// beyond the newest position are zero-filled, so stale page contents never reach a product.
//
// Prefill: one block per group of consecutive tokens of a query tile (blockIdx.y) and per group of 64 heads.
// Decode: one block per token, head group and key split; with more than one split the blocks leave unnormalised
// partial sums (float32) with their maximum and sum, and a second kernel combines them.  A learned sink per head
// joins the denominator once (in the combine when there are splits).
#include "common.cuh"

namespace cpi {
namespace lat {

constexpr int BM_MAX = 64, BN = 32, SLD = BN + 8;      // a block has RG groups of 16 query rows (1, 2 or 4), 64 threads a group
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16* q;       // [T, H, row]
  const __nv_bfloat16* cache;   // [pages, 1, page_size, row]
  __nv_bfloat16* out;           // [H T, rank] head-major (row h T + t)
  float* part_o;                // [T, H, splits, rank]   (splits > 1)
  float* part_ml;               // [T, H, splits, 2]
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  const int* tile_tok0; const int* tile_rows;      // null: tile i is token i alone
  const float* sink;            // [H] or null
  int n_tokens, n_heads, row, rank;
  int heads_per_group, tokens_per_block, n_splits;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int NT, bool FULL, int RG>
__global__ void __launch_bounds__(64 * RG, 1) latent_attention_kernel(Params p) {
  constexpr int BM = 16 * RG, THREADS = 64 * RG;
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.n_heads, HG = p.heads_per_group, row = p.row, rank = p.rank;
  const int LD = row + 8;                                        // padded shared-memory row, in elements
  int tok0, ntok, split = 0;
  if (p.tile_tok0 != nullptr) {
    const int off = blockIdx.y * p.tokens_per_block, rows = p.tile_rows[blockIdx.x];
    if (off >= rows) return;
    tok0 = p.tile_tok0[blockIdx.x] + off;
    ntok = min(p.tokens_per_block, rows - off);
  } else {
    tok0 = blockIdx.x;
    ntok = 1;
    split = blockIdx.y;
  }
  const int hg0 = blockIdx.z * HG, nh = min(HG, H - hg0);
  const int n_rows = ntok * HG;                                  // rows at and after this one are empty

  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* KVs = Qs + (size_t)BM * LD;
  float* Ss = reinterpret_cast<float*>(KVs + (size_t)2 * BN * LD);
  int* qpos_s = reinterpret_cast<int*>(Ss + BM * SLD);

  const int* table = p.page_table + (size_t)p.seq_slot[p.token_seq[tok0]] * p.max_blocks;
  const int last_pos = p.token_pos[tok0 + ntok - 1];
  const int n_kv_tiles = last_pos / BN + 1;
  const int per_split = (n_kv_tiles + p.n_splits - 1) / p.n_splits;
  const int t_begin = split * per_split, t_end = min(n_kv_tiles, t_begin + per_split);
  const int chunks = row >> 3;                                   // 16-byte pieces of a row

  // ---- queries: row m is token tok0 + m / HG, head hg0 + m % HG
  for (int m = warp; m < BM; m += THREADS / 32) {
    const int tk = m / HG, hh = m % HG;
    const bool valid = tk < ntok && hh < nh;
    __nv_bfloat16* dst = Qs + (size_t)m * LD;
    if (valid) {
      const __nv_bfloat16* src = p.q + ((size_t)(tok0 + tk) * H + hg0 + hh) * row;
      for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 8, src + c * 8);
    } else {
      for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    }
    if (lane == 0) qpos_s[m] = valid ? p.token_pos[tok0 + tk] : -1;
  }
  auto load_kv = [&](int tile, int buf) {
    __nv_bfloat16* base = KVs + (size_t)buf * BN * LD;
    for (int r = warp; r < BN; r += THREADS / 32) {
      const int kpos = tile * BN + r;
      __nv_bfloat16* dst = base + (size_t)r * LD;
      if (kpos <= last_pos) {
        const int page = table[kpos / p.page_size];
        const __nv_bfloat16* src = p.cache + ((size_t)page * p.page_size + kpos % p.page_size) * row;
        for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 8, src + c * 8);
      } else {
        for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (t_begin < t_end) load_kv(t_begin, 0);
  cp_async_commit();

  const int rg = warp % RG, ch = warp / RG;
  const int g = lane >> 2, t4 = lane & 3;
  const bool active = rg * 16 < n_rows;
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int col_base = ch * NT * 8;

  for (int it = t_begin; it < t_end; ++it) {
    const int buf = (it - t_begin) & 1;
    cp_async_wait_all();
    __syncthreads();                       // tile `it` (and the queries) have landed; the tile before is done with
    if (it + 1 < t_end) load_kv(it + 1, buf ^ 1);
    cp_async_commit();
    const __nv_bfloat16* KV = KVs + (size_t)buf * BN * LD;
    const int kv0 = it * BN;
    if (active) {
      // two k-steps a turn on accumulators of their own (four independent chains), the fragments of the next
      // turn loaded before the products of this one
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __nv_bfloat16* qa = Qs + (size_t)(rg * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
      const __nv_bfloat16* kb = KV + (size_t)(ch * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + ((lane >> 3) & 1) * 8;
      uint32_t a0[4], b0[4], a1[4], b1[4];
      const int pairs_end = row & ~31;
      ldsm_x4(a0, qa); ldsm_x4(b0, kb);                            // row >= 16: the first k-step is always there
      for (int kk = 0; kk < pairs_end; kk += 32) {
        ldsm_x4(a1, qa + kk + 16); ldsm_x4(b1, kb + kk + 16);
        mma_bf16(s[0], a0, b0[0], b0[1]);
        mma_bf16(s[1], a0, b0[2], b0[3]);
        if (kk + 32 < row) { ldsm_x4(a0, qa + kk + 32); ldsm_x4(b0, kb + kk + 32); }
        mma_bf16(s2[0], a1, b1[0], b1[1]);
        mma_bf16(s2[1], a1, b1[2], b1[3]);
      }
      if (pairs_end < row) {                                       // an odd number of k-steps: the last one is loaded
        mma_bf16(s[0], a0, b0[0], b0[1]);
        mma_bf16(s[1], a0, b0[2], b0[3]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) { s[0][u] += s2[0][u]; s[1][u] += s2[1][u]; }
      const int r0 = rg * 16 + g, qp0 = qpos_s[r0], qp1 = qpos_s[r0 + 8];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = ch * 16 + j * 8 + 2 * t4, kp = kv0 + col;
        float2 v0, v1;
        v0.x = kp <= qp0 ? s[j][0] * p.scale_log2 : -INFINITY;
        v0.y = kp + 1 <= qp0 ? s[j][1] * p.scale_log2 : -INFINITY;
        v1.x = kp <= qp1 ? s[j][2] * p.scale_log2 : -INFINITY;
        v1.y = kp + 1 <= qp1 ? s[j][3] * p.scale_log2 : -INFINITY;
        *reinterpret_cast<float2*>(Ss + r0 * SLD + col) = v0;
        *reinterpret_cast<float2*>(Ss + (r0 + 8) * SLD + col) = v1;
      }
    }
    if (active) {
      // the scores of 16 rows pass between the two warps of the row group only: a barrier of their own
      asm volatile("bar.sync %0, 64;" ::"r"(1 + rg) : "memory");
      uint32_t pa[BN / 16][4];
      float alpha[2];
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const float* sr = Ss + (rg * 16 + g + hrow * 8) * SLD + 2 * t4;
        float2 v[BN / 8];
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) v[c] = *reinterpret_cast<const float2*>(sr + c * 8);
        float mx = v[0].x;
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) mx = fmaxf(mx, fmaxf(v[c].x, v[c].y));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[hrow], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        alpha[hrow] = exp2f(m_run[hrow] - m_safe);
        m_run[hrow] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) {
          const float e0 = exp2f(v[c].x - m_safe), e1 = exp2f(v[c].y - m_safe);
          sum += e0 + e1;
          // columns 8 c + 2 t4: k-step c / 2, low or high half c % 2; rows g (registers 0, 2) and g + 8 (1, 3)
          pa[c >> 1][(c & 1) * 2 + hrow] = pack_bf16(e0, e1);
        }
        l_run[hrow] = l_run[hrow] * alpha[hrow] + sum;
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {      // a maximum of the warp's rows has grown
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
          o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
      }
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
        const __nv_bfloat16* vb = KV + (size_t)(ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + col_base + (lane >> 4) * 8;
        if (FULL) {                          // every column of the warp is a value column: nothing to ask per pair
          uint32_t b[2][4];
          ldsm_x4_trans(b[0], vb);
#pragma unroll
          for (int i = 0; i < NT; i += 2) {
            if (i + 2 < NT) ldsm_x4_trans(b[((i >> 1) + 1) & 1], vb + (i + 2) * 8);
            mma_bf16(o[i], pa[ks], b[(i >> 1) & 1][0], b[(i >> 1) & 1][1]);
            mma_bf16(o[i + 1], pa[ks], b[(i >> 1) & 1][2], b[(i >> 1) & 1][3]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < NT; i += 2) {
            if (col_base + i * 8 < rank) {
              uint32_t b[4];
              ldsm_x4_trans(b, vb + i * 8);
              mma_bf16(o[i], pa[ks], b[0], b[1]);
              mma_bf16(o[i + 1], pa[ks], b[2], b[3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait_all();
  if (!active) return;

  // ---- the end: row sums over the four lanes that share a row, the sink, the division
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    l_run[hrow] += __shfl_xor_sync(0xffffffffu, l_run[hrow], 1);
    l_run[hrow] += __shfl_xor_sync(0xffffffffu, l_run[hrow], 2);
  }
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int m = rg * 16 + g + hrow * 8;
    const int tk = m / HG, hh = m % HG;
    if (tk >= ntok || hh >= nh) continue;
    const int tok = tok0 + tk, head = hg0 + hh;
    if (p.n_splits == 1) {
      float l = l_run[hrow];
      if (p.sink != nullptr) {
        const float sk = p.sink[head] * kLog2e;
        // with no key in reach the sink alone is the denominator, and the output is zero
        l += m_run[hrow] == -INFINITY ? 1.f : exp2f(sk - m_run[hrow]);
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)head * p.n_tokens + tok) * rank;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int col = col_base + i * 8 + 2 * t4;
        if (col < rank)
          *reinterpret_cast<__nv_bfloat162*>(dst + col) =
              __floats2bfloat162_rn(o[i][hrow * 2] * inv, o[i][hrow * 2 + 1] * inv);
      }
    } else {
      const size_t slot = ((size_t)tok * H + head) * p.n_splits + split;
      float* dst = p.part_o + slot * rank;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int col = col_base + i * 8 + 2 * t4;
        if (col < rank) *reinterpret_cast<float2*>(dst + col) = make_float2(o[i][hrow * 2], o[i][hrow * 2 + 1]);
      }
      if (ch == 0 && t4 == 0) {
        p.part_ml[slot * 2] = m_run[hrow];
        p.part_ml[slot * 2 + 1] = l_run[hrow];
      }
    }
  }
}

// out[h T + t] = sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)),  M = max_s m_s
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* part_o, const float* part_ml,
                                                             __nv_bfloat16* out, const float* sink, int n_tokens,
                                                             int n_heads, int n_splits, int rank) {
  pdl_launch_dependents();
  __shared__ float w_s[64];
  __shared__ float inv_s;
  pdl_wait();
  const int tok = blockIdx.x / n_heads, head = blockIdx.x % n_heads;
  const size_t slot0 = (size_t)blockIdx.x * n_splits;
  if (threadIdx.x < 32) {
    float M = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += 32) M = fmaxf(M, part_ml[(slot0 + s) * 2]);
    M = warp_max(M);
    float L = 0.f;
    for (int s = threadIdx.x; s < n_splits; s += 32) {
      const float m = part_ml[(slot0 + s) * 2];
      const float w = (M == -INFINITY || m == -INFINITY) ? 0.f : exp2f(m - M);
      w_s[s] = w;
      L = fmaf(w, part_ml[(slot0 + s) * 2 + 1], L);
    }
    L = warp_sum(L);
    if (sink != nullptr) L += M == -INFINITY ? 1.f : exp2f(sink[head] * kLog2e - M);
    if (threadIdx.x == 0) inv_s = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  const float inv = inv_s;
  __nv_bfloat16* dst = out + ((size_t)head * n_tokens + tok) * rank;
  // four columns a thread (rank is a multiple of 16); every split's block has written its partial row (zeros when
  // it had no keys), so the loads need no condition and eight of them are in flight
  for (int c = threadIdx.x * 4; c < rank; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* src = part_o + slot0 * rank + c;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + (size_t)s * rank);
      const float w = w_s[s];
      acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
      acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    *reinterpret_cast<__nv_bfloat162*>(dst + c + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  }
}

constexpr int kMaxSplits = 64, kMaxRow = 640, kMaxRank = 512;

}  // namespace lat
}  // namespace cpi

using namespace cpi;

extern "C" int cpi_latent_attention_supported(int row, int rank) {
  return row % 16 == 0 && rank % 16 == 0 && rank >= 16 && rank <= lat::kMaxRank && rank <= row && row <= lat::kMaxRow;
}

extern "C" int cpi_latent_attention_max_splits() { return lat::kMaxSplits; }

static int lat_row_groups(int n_heads, bool runs) {
  const int most = n_heads < lat::BM_MAX ? n_heads : lat::BM_MAX;
  return runs || most > 32 ? 4 : most > 16 ? 2 : 1;
}
static size_t lat_smem(int bm, int row) {
  return (size_t)(bm + 2 * lat::BN) * (row + 8) * sizeof(__nv_bfloat16) + (size_t)bm * lat::SLD * sizeof(float)
         + bm * sizeof(int);
}

// q [T, H, row] bfloat16; cache [pages, 1, page_size, row] bfloat16; out [H T, rank] bfloat16, head-major.
// tile_tok0 / tile_rows (n_tiles of them, of at most max_tile_rows tokens): runs of consecutive tokens of one
// sequence; null: every token is a run of its own, and the keys of a token are divided over n_splits blocks
// (part_o float32 [T, H, n_splits, rank] and part_ml float32 [T, H, n_splits, 2] are then needed).
extern "C" int cpi_latent_attention(const void* q, const void* cache, void* out, float* part_o, float* part_ml,
                                    const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                    const int* token_pos, const int* seq_slot, const int* tile_tok0,
                                    const int* tile_rows, int n_tiles, int max_tile_rows, const float* sink,
                                    int n_tokens, int n_heads, int row, int rank, int n_splits, float scale,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(cpi_latent_attention_supported(row, rank), "latent_attention: rows of %d with a latent of %d are not "
              "supported (multiples of 16, a latent of at most %d, a row of at most %d)", row, rank, lat::kMaxRank,
              lat::kMaxRow);
  CPI_REQUIRE(n_heads >= 1 && page_size >= 1 && n_splits >= 1 && n_splits <= lat::kMaxSplits,
              "latent_attention: bad sizes heads=%d page=%d splits=%d", n_heads, page_size, n_splits);
  CPI_REQUIRE(tile_tok0 == nullptr || n_splits == 1, "latent_attention: key splits go with single-token runs");
  CPI_REQUIRE(n_splits == 1 || (part_o != nullptr && part_ml != nullptr), "latent_attention: key splits need the "
              "buffers of the partial sums");
  lat::Params p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.cache = reinterpret_cast<const __nv_bfloat16*>(cache);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml;
  p.page_table = page_table; p.max_blocks = max_blocks; p.page_size = page_size;
  p.token_seq = token_seq; p.token_pos = token_pos; p.seq_slot = seq_slot;
  p.tile_tok0 = tile_tok0; p.tile_rows = tile_rows;
  p.sink = sink;
  p.n_tokens = n_tokens; p.n_heads = n_heads; p.row = row; p.rank = rank;
  // rows of a block: 64 in a prompt; for single tokens no more groups of 16 than the heads fill, so that the
  // blocks are small, two share a multiprocessor and the keys can be divided further
  // single tokens: small blocks (several to a multiprocessor) only when there are more blocks than multiprocessors;
  // below that a block of eight warps is faster, its idle warps fetching the tiles
  const int hg64 = (n_heads + lat::BM_MAX - 1) / lat::BM_MAX;
  const bool crowded = tile_tok0 == nullptr && (long)n_tokens * n_splits * hg64 > sm_count();
  const int rg = crowded ? lat_row_groups(n_heads, false) : 4;
  const int bm = 16 * rg;
  p.heads_per_group = n_heads < bm ? n_heads : bm;
  p.tokens_per_block = bm / p.heads_per_group;
  p.n_splits = n_splits;
  p.scale_log2 = scale * lat::kLog2e;
  const int head_groups = (n_heads + p.heads_per_group - 1) / p.heads_per_group;
  dim3 grid;
  if (tile_tok0 != nullptr) {
    CPI_REQUIRE(n_tiles >= 1 && max_tile_rows >= 1, "latent_attention: %d runs of %d tokens", n_tiles, max_tile_rows);
    grid = dim3(n_tiles, (max_tile_rows + p.tokens_per_block - 1) / p.tokens_per_block, head_groups);
  } else {
    grid = dim3(n_tokens, n_splits, head_groups);
  }
  const size_t smem = lat_smem(bm, row);
#define CPI_LAT_LAUNCH_RG(NT, RG)                                                                              \
  do {                                                                                                         \
    auto kernel = rank == NT * 16 ? lat::latent_attention_kernel<NT, true, RG>                                 \
                                  : lat::latent_attention_kernel<NT, false, RG>;                               \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
    cpi::launch_pdl(kernel, grid, dim3(64 * RG), smem, stream, p);                                             \
  } while (0)
#define CPI_LAT_LAUNCH(NT)                                                                                     \
  do {                                                                                                         \
    if (rg == 4) CPI_LAT_LAUNCH_RG(NT, 4);                                                                     \
    else if (rg == 2) CPI_LAT_LAUNCH_RG(NT, 2);                                                                \
    else CPI_LAT_LAUNCH_RG(NT, 1);                                                                             \
  } while (0)
  if (rank <= 128) CPI_LAT_LAUNCH(8);
  else if (rank <= 256) CPI_LAT_LAUNCH(16);
  else CPI_LAT_LAUNCH(32);
#undef CPI_LAT_LAUNCH_RG
#undef CPI_LAT_LAUNCH
  if (check_launch("latent_attention")) return 1;
  if (n_splits > 1) {
    cpi::launch_pdl(lat::latent_combine_kernel, dim3(n_tokens * n_heads), dim3(128), 0, stream,
                    (const float*)part_o, (const float*)part_ml, reinterpret_cast<__nv_bfloat16*>(out), sink, n_tokens,
                    n_heads, n_splits, rank);
    return check_launch("latent_combine");
  }
  return 0;
}
