// Latent attention on the tensor cores (bfloat16): prompts and decode steps with one kernel.
//
// A query row is a (token, head) pair; all heads of a token read the same cached rows [rank latent | rot shared
// key part], so a block takes 16 * MT consecutive rows of one sequence (row = token * H + head: in a decode step
// the heads of the sequence's one token, in a prompt a few tokens with all their heads) and walks the sequence's
// pages once for all of them.  A page (64 positions) is one key tile AND one value tile: the scores use the whole
// row, the weighted sum its first `rank` columns, so a tile is copied to shared memory once (cp.async, two stages).
//
//   warp (i, j), i < MT, j < 4:  S[16 rows of tile i][keys 16 j .. 16 j + 15] = Q K^T   (mma.sync m16n8k16, k = rank + rot)
//   the four j-warps of a row tile exchange their row maxima through shared memory, write P = 2^(S - max) in bfloat16
//   warp (i, j):                 O[16 rows][columns j rank/4 .. (j+1) rank/4) += P V    (V = the tile, read transposed)
//
// The softmax sink of a head is the start value of its rows' running maximum and sum in the block that takes the first
// part of the key range.  The key range of a sequence may be cut into `n_splits` parts (decode steps, to fill the GPU):
// each part leaves (max, sum, unnormalised O) per row, and `latent_merge` adds the parts.  With one part the kernel
// writes the result itself.
//
// Sizes: rank in {64, 128, 256, 512}, rot a multiple of 16 (0 allowed); everything else goes to the plain kernel.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BN 64  // keys per tile = page size

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// q_cat: [T, H, Dk] bf16.  pages: [n_pages, 64, Dk].  For sequence s: tokens seq_start[s] .. seq_start[s+1]-1 at positions
// seq_pos0[s] + 0, 1, ...  part_o: [rows_total, n_splits, RANK], part_ml: [rows_total, n_splits, 2] (only with n_splits > 1).
template <int RANK, int MT>
__global__ void __launch_bounds__(128 * MT)
latent_attn_mma_kernel(const bf16* __restrict__ q_cat, const bf16* __restrict__ pages, const int* __restrict__ block_table,
                       int table_width, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                       const float* __restrict__ sink, bf16* __restrict__ out, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int H, int rot, int window, float scale_log2, int n_splits) {
  constexpr int NT = 128 * MT;
  constexpr int BM = 16 * MT;
  constexpr int OW = RANK / 4;  // result columns per warp
  const int Dk = RANK + rot;
  const int STRIDE = Dk + 8;  // 16 bytes of padding per row: ldmatrix without bank conflicts
  constexpr int PSTRIDE = BN + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [BM][STRIDE]
  bf16* k_s0 = q_s + (size_t)BM * STRIDE;          // two stages [BN][STRIDE]
  bf16* k_s1 = k_s0 + (size_t)BN * STRIDE;
  bf16* p_s = k_s1 + (size_t)BN * STRIDE;          // [BM][PSTRIDE]
  float* red = reinterpret_cast<float*>(p_s + (size_t)BM * PSTRIDE);  // [BM][4] row maxima of the four key quarters, then sums

  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x, split = blockIdx.z;
  const int tok0 = seq_start[s];
  const int n_rows = (seq_start[s + 1] - tok0) * H;
  const int row0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;  // the last rows, which see the most keys, start first
  if (row0 >= n_rows) return;
  const int pos0 = seq_pos0[s];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wi = warp >> 2, wj = warp & 3;
  const int g = lane >> 2, t4 = lane & 3;
  const int rows_here = min(BM, n_rows - row0);
  const int first_pos = pos0 + row0 / H, last_pos = pos0 + (row0 + rows_here - 1) / H;
  const int lowest_key = (window != 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
  // this block's part of the tiles lowest_key / 64 .. last_pos / 64
  const int t_lo = lowest_key / BN, t_hi = last_pos / BN;
  const int n_tiles = t_hi - t_lo + 1;
  const int per = (n_tiles + n_splits - 1) / n_splits;
  const int tile_lo = t_lo + split * per, tile_hi = min(t_hi, tile_lo + per - 1);
  const size_t grow0 = (size_t)tok0 * H + row0;  // first row of this block among all rows of the step

  const int* table = block_table + (size_t)s * table_width;
  const int chunks = Dk >> 3;
  auto load_tile = [&](bf16* dst, int tile) {
    const bf16* src = pages + (size_t)table[tile] * BN * Dk;
    for (int c = tid; c < BN * chunks; c += NT) {
      const int r = c / chunks, cc = c - r * chunks;
      cp_async_16(dst + (size_t)r * STRIDE + cc * 8, src + (size_t)r * Dk + cc * 8);
    }
  };
  if (tile_lo <= tile_hi) {
    // queries (rows past the end are zeros) and the first tile
    for (int c = tid; c < BM * chunks; c += NT) {
      const int r = c / chunks, cc = c - r * chunks;
      if (r < rows_here) cp_async_16(q_s + (size_t)r * STRIDE + cc * 8, q_cat + (grow0 + r) * Dk + cc * 8);
      else *reinterpret_cast<uint4*>(q_s + (size_t)r * STRIDE + cc * 8) = make_uint4(0, 0, 0, 0);
    }
    load_tile(k_s0, tile_lo);
  }
  cp_async_commit();

  float o_acc[OW / 8][4];
#pragma unroll
  for (int i = 0; i < OW / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  // rows of this thread: wi * 16 + g and + 8
  int qpos[2];
  float m_run[2], l_run[2];  // l_run: this thread's share of its key quarter's sum
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + wi * 16 + g + 8 * r;
    const bool live = row < n_rows;
    qpos[r] = live ? pos0 + row / H : -1;
    const bool with_sink = sink != nullptr && split == 0 && live;
    m_run[r] = with_sink ? sink[row % H] * 1.4426950408889634f : -INFINITY;
    l_run[r] = (with_sink && wj == 0 && t4 == 0) ? 1.f : 0.f;
  }

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    bf16* k_s = buf ? k_s1 : k_s0;
    if (tile + 1 <= tile_hi) {
      load_tile(buf ? k_s0 : k_s1, tile + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // ---- S for this warp's 16 rows and its quarter of the keys
    float s_acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
    const bf16* qa = q_s + (size_t)(wi * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + 8 * (lane >> 4);
    const bf16* kb = k_s + (size_t)(wj * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + 8 * ((lane >> 3) & 1);
    const int ksteps = Dk >> 4;
#pragma unroll 4
    for (int kk = 0; kk < ksteps; ++kk) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, qa + kk * 16);
      ldmatrix_x4(b, kb + kk * 16);
      mma_bf16(s_acc[0], a, b[0], b[1]);
      mma_bf16(s_acc[1], a, b[2], b[3]);
    }
    // ---- scale to base-2 exponents, mask, this quarter's row maxima
    const int key0 = tile * BN + wj * 16;
    float qmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int key = key0 + n * 8 + 2 * t4 + (e & 1);
        const bool seen = key <= qpos[r] && (window == 0 || qpos[r] - key < window);
        const float v = seen ? s_acc[n][e] * scale_log2 : -INFINITY;
        s_acc[n][e] = v;
        qmax[r] = fmaxf(qmax[r], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = qmax[r];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      if (t4 == 0) red[(wi * 16 + g + 8 * r) * 4 + wj] = mx;
    }
    __syncthreads();
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float4 q4 = *reinterpret_cast<const float4*>(red + (wi * 16 + g + 8 * r) * 4);
      const float m_new = fmaxf(m_run[r], fmaxf(fmaxf(q4.x, q4.y), fmaxf(q4.z, q4.w)));
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // a row that has seen nothing yet: nothing becomes NaN
      alpha[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
    // ---- P in bfloat16 into shared memory; the sums are taken from the rounded values' 32-bit originals
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = exp2f(s_acc[n][e] - m_use[e >> 1]);
        l_run[e >> 1] += p[e];
      }
      bf16* pr = p_s + (size_t)(wi * 16 + g) * PSTRIDE + wj * 16 + n * 8 + 2 * t4;
      *reinterpret_cast<__nv_bfloat162*>(pr) = __floats2bfloat162_rn(p[0], p[1]);
      *reinterpret_cast<__nv_bfloat162*>(pr + 8 * PSTRIDE) = __floats2bfloat162_rn(p[2], p[3]);
    }
#pragma unroll
    for (int i = 0; i < OW / 8; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1];
      o_acc[i][3] *= alpha[1];
    }
    __syncthreads();
    // ---- O += P V for this warp's columns
    const bf16* pa = p_s + (size_t)(wi * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * PSTRIDE + 8 * (lane >> 4);
    const bf16* vb = k_s + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + wj * OW + 8 * (lane >> 4);
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, pa + kk * 16);
#pragma unroll
      for (int dp = 0; dp < OW / 16; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vb + (size_t)kk * 16 * STRIDE + dp * 16);
        mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
        mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // every warp is done with this stage, P and the maxima before they are written again
  }

  // ---- the rows' sums over the quad and over the four key quarters
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t4 == 0) red[(wi * 16 + g + 8 * r) * 4 + wj] = l;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int lrow = wi * 16 + g + 8 * r;
    if (lrow >= rows_here) continue;
    const float4 q4 = *reinterpret_cast<const float4*>(red + lrow * 4);
    const float l = (q4.x + q4.y) + (q4.z + q4.w);
    if (n_splits == 1) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* o = out + (grow0 + lrow) * RANK + wj * OW;
#pragma unroll
      for (int n = 0; n < OW / 8; ++n)
        *reinterpret_cast<__nv_bfloat162*>(o + n * 8 + 2 * t4) = __floats2bfloat162_rn(o_acc[n][2 * r] * inv, o_acc[n][2 * r + 1] * inv);
    } else {
      float* o = part_o + ((grow0 + lrow) * n_splits + split) * RANK + wj * OW;
#pragma unroll
      for (int n = 0; n < OW / 8; ++n) *reinterpret_cast<float2*>(o + n * 8 + 2 * t4) = make_float2(o_acc[n][2 * r], o_acc[n][2 * r + 1]);
      if (wj == 0 && t4 == 0) {
        float* ml = part_ml + ((grow0 + lrow) * n_splits + split) * 2;
        ml[0] = m_run[r];
        ml[1] = l;
      }
    }
  }
}

// out[row] = sum_i 2^(m_i - M) o_i / sum_i 2^(m_i - M) l_i over the parts of the key range, parts in their order.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    int n_splits, int rank) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * n_splits * 2;
  float M = -INFINITY;
  for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
  float l = 0.f;
  for (int i = 0; i < n_splits; ++i) l += (ml[2 * i] == -INFINITY) ? 0.f : exp2f(ml[2 * i] - M) * ml[2 * i + 1];
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float v = 0.f;
    for (int i = 0; i < n_splits; ++i)
      if (ml[2 * i] != -INFINITY) v += exp2f(ml[2 * i] - M) * part_o[(row * n_splits + i) * rank + d];
    out[row * rank + d] = __float2bfloat16_rn(v * inv);
  }
}

RL_API long long rl_latent_attn_mma_scratch_floats(long long rows, int rank, int n_splits) {
  return n_splits > 1 ? rows * n_splits * (rank + 2) : 0;
}

// 1 if the kernel takes these sizes, else 0
RL_API int rl_latent_attn_mma_takes(int rank, int rot) {
  return (rank == 64 || rank == 128 || rank == 256 || rank == 512) && rot >= 0 && rot % 16 == 0 && rot <= 256;
}

template <int RANK, int MT>
static int launch_latent(const bf16* q_cat, const bf16* pages, const int* block_table, int table_width, const int* seq_start,
                         const int* seq_pos0, const float* sink, bf16* out, float* scratch, long long rows_total, int n_seqs,
                         int max_rows, int H, int rot, int window, float scale, int n_splits, cudaStream_t stream) {
  const int Dk = RANK + rot, BM = 16 * MT;
  const size_t smem = (size_t)(BM + 2 * BN) * (Dk + 8) * sizeof(bf16) + (size_t)BM * (BN + 8) * sizeof(bf16) + (size_t)BM * 4 * sizeof(float);
  auto kern = latent_attn_mma_kernel<RANK, MT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(8, "latent_attn_mma: cannot get %zu bytes of shared memory", smem);
  }
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + rows_total * n_splits * RANK : nullptr;
  dim3 grid(n_seqs, (max_rows + BM - 1) / BM, n_splits);
  RL_LAUNCH_CHECK(rl_launch<false>(kern, grid, 128 * MT, smem, stream, q_cat, pages, block_table, table_width, seq_start, seq_pos0,
                                   sink, out, part_o, part_ml, H, rot, window, scale * 1.4426950408889634f, n_splits));
  if (n_splits > 1)
    RL_LAUNCH_CHECK(rl_launch<false>(latent_merge_kernel, (unsigned)rows_total, RANK >= 256 ? 128 : 64, 0, stream, (const float*)part_o,
                                     (const float*)part_ml, out, n_splits, RANK));
  return 0;
}

// max_rows: the most rows (tokens * H) any sequence brings.  rows_total: all rows of the step.
RL_API int rl_latent_attn_mma(const void* q_cat, const void* pages, const int* block_table, int table_width, const int* seq_start,
                              const int* seq_pos0, const float* sink, void* out, float* scratch, long long rows_total, int n_seqs,
                              int max_rows, int H, int rank, int rot, int page_size, int window, float scale, int n_splits,
                              cudaStream_t stream) {
  if (n_seqs <= 0 || max_rows <= 0 || H <= 0 || rows_total <= 0 || n_splits <= 0)
    RL_REFUSE(1, "latent_attn_mma: S=%d rows=%d H=%d splits=%d", n_seqs, max_rows, H, n_splits);
  if (!rl_latent_attn_mma_takes(rank, rot)) RL_REFUSE(2, "latent_attn_mma: rank %d / rot %d are not sizes this kernel is built for", rank, rot);
  if (page_size != BN) RL_REFUSE(3, "latent_attn_mma: page size %d, this kernel is built for %d", page_size, BN);
  if (window < 0) RL_REFUSE(4, "latent_attn_mma: negative window");
  if (n_splits > 1 && scratch == nullptr) RL_REFUSE(5, "latent_attn_mma: %d parts but no scratch", n_splits);
  if (n_splits > 65535 || (max_rows + 15) / 16 > 65535) RL_REFUSE(6, "latent_attn_mma: the grid does not take these sizes");
  const bool two = max_rows > 16;  // a decode step of a model with 16 heads or fewer: one row tile
#define RL_LA(R)                                                                                                                  \
  do {                                                                                                                            \
    if (two)                                                                                                                      \
      return launch_latent<R, 2>((const bf16*)q_cat, (const bf16*)pages, block_table, table_width, seq_start, seq_pos0, sink,    \
                                 (bf16*)out, scratch, rows_total, n_seqs, max_rows, H, rot, window, scale, n_splits, stream);     \
    return launch_latent<R, 1>((const bf16*)q_cat, (const bf16*)pages, block_table, table_width, seq_start, seq_pos0, sink,      \
                               (bf16*)out, scratch, rows_total, n_seqs, max_rows, H, rot, window, scale, n_splits, stream);       \
  } while (0)
  if (rank == 64) RL_LA(64);
  if (rank == 128) RL_LA(128);
  if (rank == 256) RL_LA(256);
  RL_LA(512);
#undef RL_LA
}
