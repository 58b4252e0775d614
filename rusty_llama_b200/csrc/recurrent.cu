// Mixers whose memory is a fixed-size state per sequence instead of a growing cache, and the row kernels around them.
// The state is 32-bit and lives in the cache's state records, state[slot]; a step reads the record of each of its
// sequences, runs the sequence's tokens through it in order and writes it back.  Everything that enters a recurrence
// is computed in 32-bit from the projections, which come in the run's element type.
//
//   decay_attn   linear attention with a constant decay per head:
//                  S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t      (S is [dim, vdim] per head)
//                with an optional activation (silu) applied to the projected q, k, v as they are read.
//   rms_gate     y = x / sqrt(mean(x^2) + eps) * w * sigmoid(g) * c over whole rows (x 32-bit), the step between
//                decay_attn and the output projection.
//   min_gru      element by element  S_t = (1 - z_t) S_(t-1) + z_t c_t,  z = sigmoid(a + b_z),
//                c = u + 1/2 where u >= 0, else sigmoid(u), u = x + b_x;  result S_t * silu(g_t) * c_out.
//   unary_act    y = f(x) element by element; f = relu(x)^2.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

__device__ __forceinline__ float logistic(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * logistic(x); }

// ---------------------------------------------------------------- linear attention with decay
// A block owns 32 columns of one head's state for one sequence: lane = column, warp w holds rows 32 w .. 32 w + 31 of
// those columns in registers.  Tokens are taken DA_TOK at a time: their q, k (whole head) and v (the block's columns)
// go to shared memory, every warp runs the tokens through its rows, and the warps' partial results are added in warp
// order.  The order of every sum is fixed by the sizes alone.
#define DA_TOK 16

template <typename T>
__global__ void decay_attn_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
                                  const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ slot_ids,
                                  const int* __restrict__ seq_start, float* __restrict__ out, int out_stride, int H, int dim, int vdim,
                                  int act) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * 32;
  const int col = col0 + lane;
  const bool col_ok = col < vdim;
  float* q_s = sm;                      // [DA_TOK][dim]
  float* k_s = q_s + DA_TOK * dim;      // [DA_TOK][dim]
  float* v_s = k_s + DA_TOK * dim;      // [DA_TOK][32]
  float* part = v_s + DA_TOK * 32;      // [nw][DA_TOK][32]
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  const float lam = decay[h];
  float* st = state + (((size_t)slot_ids[s] * H + h) * dim) * vdim;
  float S[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = w * 32 + r;
    S[r] = (row < dim && col_ok) ? st[(size_t)row * vdim + col] : 0.f;
  }
  for (int base = t0; base < t1; base += DA_TOK) {
    const int n = min(DA_TOK, t1 - base);
    for (int idx = threadIdx.x; idx < n * dim; idx += blockDim.x) {
      const int j = idx / dim, i = idx - j * dim;
      const size_t at = (size_t)(base + j) * in_stride + (size_t)h * dim + i;
      float qv = to_f32(q[at]), kv = to_f32(k[at]);
      if (act) {
        qv = silu_f(qv);
        kv = silu_f(kv);
      }
      q_s[j * dim + i] = qv;
      k_s[j * dim + i] = kv;
    }
    for (int idx = threadIdx.x; idx < n * 32; idx += blockDim.x) {
      const int j = idx >> 5, c = idx & 31;
      float vv = 0.f;
      if (col0 + c < vdim) {
        vv = to_f32(v[(size_t)(base + j) * in_stride + (size_t)h * vdim + col0 + c]);
        if (act) vv = silu_f(vv);
      }
      v_s[idx] = vv;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float vj = v_s[j * 32 + lane];
      const float* kj = k_s + j * dim + w * 32;
      const float* qj = q_s + j * dim + w * 32;
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        if (w * 32 + r < dim) {
          S[r] = lam * S[r] + kj[r] * vj;
          o += S[r] * qj[r];
        }
      }
      part[(w * DA_TOK + j) * 32 + lane] = o;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * 32; idx += blockDim.x) {
      const int j = idx >> 5, c = idx & 31;
      if (col0 + c < vdim) {
        float o = 0.f;
        for (int ww = 0; ww < nw; ++ww) o += part[(ww * DA_TOK + j) * 32 + c];
        out[(size_t)(base + j) * out_stride + (size_t)h * vdim + col0 + c] = o;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = w * 32 + r;
    if (row < dim && col_ok) st[(size_t)row * vdim + col] = S[r];
  }
}

RL_API int rl_decay_attn(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* decay, float* state,
                         const int* slot_ids, const int* seq_start, float* out, int out_stride, int n_seqs, int H, int dim, int vdim,
                         int act, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || dim <= 0 || vdim <= 0) RL_REFUSE(1, "decay_attn: S=%d H=%d dim=%d vdim=%d", n_seqs, H, dim, vdim);
  if (dim > 1024) RL_REFUSE(2, "decay_attn: key size %d exceeds 1024", dim);
  if (H > 65535 || (vdim + 31) / 32 > 65535) RL_REFUSE(3, "decay_attn: %d heads or %d columns exceed the grid", H, vdim);
  const int nw = (dim + 31) / 32;
  const size_t smem = ((size_t)2 * DA_TOK * dim + DA_TOK * 32 + (size_t)nw * DA_TOK * 32) * sizeof(float);
  dim3 grid(n_seqs, H, (vdim + 31) / 32);
#define RL_DA(T)                                                                                                                  \
  do {                                                                                                                            \
    if (smem > 48 * 1024) {                                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(decay_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      if (e != cudaSuccess) RL_REFUSE(4, "decay_attn: %zu bytes of shared memory refused", smem);                                 \
    }                                                                                                                             \
    decay_attn_kernel<T><<<grid, nw * 32, smem, stream>>>((const T*)q, (const T*)k, (const T*)v, in_stride, decay, state, slot_ids, \
                                                          seq_start, out, out_stride, H, dim, vdim, act);                         \
  } while (0)
  if (dtype == RL_BF16) RL_DA(bf16);
  else if (dtype == RL_F32) RL_DA(float);
  else RL_REFUSE(5, "decay_attn: unknown dtype %d", dtype);
#undef RL_DA
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the same recurrence, chunk by chunk
// For prompts.  A sequence's tokens are cut into chunks of DC; with n tokens in a chunk, S the state before it, lam the decay:
//   U      = sum_i lam^(n-1-i) k_i v_i^T                                   (1) what the chunk adds to the state, every chunk at once
//   S_next = lam^n S + U                                                    (2) the states before every chunk, chunk after chunk
//   o_i    = lam^(i+1) S^T q_i + sum_{j<=i} lam^(i-j) (q_i . k_j) v_j       (3) the outputs, every chunk at once
// Three kernels over a scratch of one [dim, vdim] matrix per (sequence, head, chunk).  All of it is 32-bit FMA arithmetic;
// only powers of lam with exponents >= 0 occur.  The order of the sums differs from the token-by-token kernel's and depends
// on where the chunks fall, so runs that promise equal bits for every cut of a sequence keep to the other kernel.
#define DC 64       // tokens per chunk
#define DC_COLS 64  // state columns per block

// (1): grid (S * H, chunks, column tiles), 256 threads: thread (ty, tx) owns rows ty + 16 a and columns 4 tx .. 4 tx + 3.
template <typename T>
__global__ void __launch_bounds__(256)
decay_chunk_state_kernel(const T* __restrict__ k, const T* __restrict__ v, int in_stride, const float* __restrict__ decay,
                         const int* __restrict__ seq_start, float* __restrict__ scratch, int max_chunks, int H, int dim, int vdim, int act) {
  extern __shared__ float sm[];
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y, col0 = blockIdx.z * DC_COLS;
  const int t0 = seq_start[s] + c * DC;
  const int n = min(DC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  float* k_s = sm;             // [DC][dim], weighted by lam^(n-1-i)
  float* v_s = sm + DC * dim;  // [DC][DC_COLS]
  __shared__ float pw[DC];
  const float lam = decay[h];
  if (threadIdx.x < DC) pw[threadIdx.x] = powf(lam, (float)threadIdx.x);
  __syncthreads();
  if (sizeof(T) == 2 && ((dim | in_stride) & 7) == 0 && (((uintptr_t)k) & 15) == 0) {  // sixteen bytes a load
#pragma unroll 2
    for (int idx = threadIdx.x; idx < n * (dim / 8); idx += 256) {
      const int i = idx / (dim / 8), r = 8 * (idx - i * (dim / 8));
      float f[8];
      bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(k + (size_t)(t0 + i) * in_stride + (size_t)h * dim + r)), f);
      const float w = pw[n - 1 - i];
#pragma unroll
      for (int e = 0; e < 8; ++e) k_s[i * dim + r + e] = (act ? silu_f(f[e]) : f[e]) * w;
    }
  } else {
#pragma unroll 4
    for (int idx = threadIdx.x; idx < n * dim; idx += 256) {
      const int i = idx / dim, r = idx - i * dim;
      float kv = to_f32(k[(size_t)(t0 + i) * in_stride + (size_t)h * dim + r]);
      if (act) kv = silu_f(kv);
      k_s[idx] = kv * pw[n - 1 - i];
    }
  }
#pragma unroll 4
  for (int idx = threadIdx.x; idx < n * DC_COLS; idx += 256) {
    const int i = idx / DC_COLS, cc = idx - i * DC_COLS;
    float vv = 0.f;
    if (col0 + cc < vdim) {
      vv = to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + col0 + cc]);
      if (act) vv = silu_f(vv);
    }
    v_s[idx] = vv;
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float acc[16][4];
#pragma unroll
  for (int a = 0; a < 16; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
  for (int i = 0; i < n; ++i) {
    const float4 vv = *reinterpret_cast<const float4*>(v_s + i * DC_COLS + 4 * tx);
#pragma unroll
    for (int a = 0; a < 16; ++a) {
      const int r = ty + 16 * a;
      if (r < dim) {
        const float kv = k_s[i * dim + r];
        acc[a][0] += kv * vv.x;
        acc[a][1] += kv * vv.y;
        acc[a][2] += kv * vv.z;
        acc[a][3] += kv * vv.w;
      }
    }
  }
  float* u = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vdim;
#pragma unroll
  for (int a = 0; a < 16; ++a) {
    const int r = ty + 16 * a;
    if (r < dim) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = col0 + 4 * tx + e;
        if (col < vdim) u[(size_t)r * vdim + col] = acc[a][e];
      }
    }
  }
}

// (2): one thread per element of a (sequence, head)'s state; leaves in every chunk's place the state BEFORE that chunk.
__global__ void decay_chunk_scan_kernel(const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ slot_ids,
                                        const int* __restrict__ seq_start, float* __restrict__ scratch, int max_chunks, int H, int elems) {
  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int e = blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= elems) return;
  const int len = seq_start[s + 1] - seq_start[s];
  const float lam = decay[h];
  float* st = state + ((size_t)slot_ids[s] * H + h) * elems + e;
  float* u = scratch + (size_t)blockIdx.x * max_chunks * elems + e;
  float S = *st;
  const float lam_full = powf(lam, (float)DC);
  const int n_chunks = (len + DC - 1) / DC;
  for (int c0 = 0; c0 < n_chunks; c0 += 8) {  // eight chunks' additions are asked for at once, then taken in order
    float add[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < n_chunks) add[j] = __ldcg(u + (size_t)(c0 + j) * elems);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      if (c < n_chunks) {
        const int n = min(DC, len - c * DC);
        u[(size_t)c * elems] = S;
        S = (n == DC ? lam_full : powf(lam, (float)n)) * S + add[j];
      }
    }
  }
  *st = S;
}

// (3): grid as (1).  Thread (ty, tx): scores P[ty + 16 a][tx + 16 b], then outputs for rows ty + 16 a and columns 4 tx .. 4 tx + 3.
template <typename T>
__global__ void __launch_bounds__(256)
decay_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
                       const float* __restrict__ decay, const int* __restrict__ seq_start, const float* __restrict__ scratch,
                       int max_chunks, float* __restrict__ out, int out_stride, int H, int dim, int vdim, int act) {
  extern __shared__ float sm[];
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y, col0 = blockIdx.z * DC_COLS;
  const int t0 = seq_start[s] + c * DC;
  const int n = min(DC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  const int DS = dim + 1;  // rows one apart in the banks
  float* q_s = sm;                    // [DC][DS]
  float* k_s = q_s + DC * DS;         // [DC][DS]
  float* v_s = k_s + DC * DS;         // [DC][DC_COLS]
  float* p_s = v_s + DC * DC_COLS;    // [DC][DC + 1]
  float* pw = p_s + DC * (DC + 1);    // lam^0 .. lam^DC
  const float lam = decay[h];
  for (int i = threadIdx.x; i <= DC; i += 256) pw[i] = powf(lam, (float)i);
  for (int idx = threadIdx.x; idx < DC * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    float qv = 0.f, kv = 0.f;
    if (i < n) {
      const size_t at = (size_t)(t0 + i) * in_stride + (size_t)h * dim + r;
      qv = to_f32(q[at]);
      kv = to_f32(k[at]);
      if (act) {
        qv = silu_f(qv);
        kv = silu_f(kv);
      }
    }
    q_s[i * DS + r] = qv;
    k_s[i * DS + r] = kv;
  }
  for (int idx = threadIdx.x; idx < DC * DC_COLS; idx += 256) {
    const int i = idx / DC_COLS, cc = idx - i * DC_COLS;
    float vv = 0.f;
    if (i < n && col0 + cc < vdim) {
      vv = to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + col0 + cc]);
      if (act) vv = silu_f(vv);
    }
    v_s[idx] = vv;
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  {
    float p[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) p[a][0] = p[a][1] = p[a][2] = p[a][3] = 0.f;
    for (int r = 0; r < dim; ++r) {
      float qa[4], kb[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) qa[a] = q_s[(ty + 16 * a) * DS + r];
#pragma unroll
      for (int b = 0; b < 4; ++b) kb[b] = k_s[(tx + 16 * b) * DS + r];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) p[a][b] += qa[a] * kb[b];
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = ty + 16 * a, j = tx + 16 * b;
        p_s[i * (DC + 1) + j] = j <= i ? p[a][b] * pw[i - j] : 0.f;
      }
  }
  __syncthreads();
  float intra[4][4], inter[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int e = 0; e < 4; ++e) intra[a][e] = inter[a][e] = 0.f;
  for (int j = 0; j < n; ++j) {
    const float4 vv = *reinterpret_cast<const float4*>(v_s + j * DC_COLS + 4 * tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const float pv = p_s[(ty + 16 * a) * (DC + 1) + j];
      intra[a][0] += pv * vv.x;
      intra[a][1] += pv * vv.y;
      intra[a][2] += pv * vv.z;
      intra[a][3] += pv * vv.w;
    }
  }
  // the state before this chunk, this block's columns: through the keys' place in shared memory, which the scores no longer need
  // (every thread has written its scores, and the barrier above has passed)
  const float* sp = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vdim;
  float* s_s = k_s;  // [dim][DC_COLS]; DC * (dim + 1) >= dim * DC_COLS
  for (int idx = threadIdx.x; idx < dim * DC_COLS; idx += 256) {
    const int r = idx / DC_COLS, cc = idx - r * DC_COLS;
    s_s[idx] = (col0 + cc < vdim) ? sp[(size_t)r * vdim + col0 + cc] : 0.f;
  }
  __syncthreads();
  for (int r = 0; r < dim; ++r) {
    const float4 t = *reinterpret_cast<const float4*>(s_s + r * DC_COLS + 4 * tx);
    const float sv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const float qv = q_s[(ty + 16 * a) * DS + r];
#pragma unroll
      for (int e = 0; e < 4; ++e) inter[a][e] += qv * sv[e];
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = ty + 16 * a;
    if (i < n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = col0 + 4 * tx + e;
        if (col < vdim) out[(size_t)(t0 + i) * out_stride + (size_t)h * vdim + col] = intra[a][e] + pw[i + 1] * inter[a][e];
      }
    }
  }
}

// (3) on the tensor cores, for bfloat16 runs with key and value sizes up to 128: a block of four warps per (sequence, head, chunk),
// a warp per 16 tokens.  q, k, v go to shared memory as bfloat16 after their activation (they are activations of projections);
// the chunk's scores Q K^T come from mma.sync with 32-bit sums, are decayed and masked in 32-bit, and meet the values as TWO
// bfloat16 numbers each (the score rounded, and what the rounding left), so the weighted sum sees 16 digits of them; the state
// before the chunk, which is 32-bit, meets the queries the same way, as two bfloat16 halves that take the place of the chunk's
// keys and values in shared memory one after the other.
__device__ __forceinline__ void rc_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void rc_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void rc_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// a 32-bit number as two bfloat16: hi = the number rounded, lo = what the rounding left
__device__ __forceinline__ void rc_split(float v, bf16& hi, bf16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}
__device__ __forceinline__ uint32_t rc_pack(bf16 a, bf16 b) {
  __nv_bfloat162 v(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(128)
decay_chunk_out_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, int in_stride,
                           const float* __restrict__ decay, const int* __restrict__ seq_start, const float* __restrict__ scratch,
                           int max_chunks, float* __restrict__ out, int out_stride, int H, int dim, int vdim, int act) {
  constexpr int STRIDE = HD + 8;
  constexpr int KSTEPS = HD / 16;
  extern __shared__ __align__(16) unsigned char rc_smem[];
  bf16* q_s = reinterpret_cast<bf16*>(rc_smem);  // [DC][STRIDE]
  bf16* k_s = q_s + DC * STRIDE;                 // [DC][STRIDE]
  bf16* v_s = k_s + DC * STRIDE;                 // [DC][STRIDE]; k_s and v_s together later hold a half of the state, [2 DC >= HD][STRIDE]
  __shared__ float pw[DC + 1];
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y;
  const int t0 = seq_start[s] + c * DC;
  const int n = min(DC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const float lam = decay[h];
  for (int i = tid; i <= DC; i += 128) pw[i] = powf(lam, (float)i);
  const bf16 zero = __float2bfloat16_rn(0.f);
  const bool vec8 = ((dim | vdim | in_stride) & 7) == 0 && ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v)) & 15) == 0;
  if (vec8) {  // sixteen bytes a load: eight numbers of q and k, or of v, per thread and round
#pragma unroll 2
    for (int idx = tid; idx < DC * (HD / 8); idx += 128) {
      const int i = idx / (HD / 8), r = 8 * (idx - i * (HD / 8));
      float qf[8], kf[8], vf[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) qf[e] = kf[e] = vf[e] = 0.f;
      if (i < n) {
        if (r < dim) {
          const size_t at = (size_t)(t0 + i) * in_stride + (size_t)h * dim + r;
          bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(q + at)), qf);
          bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(k + at)), kf);
        }
        if (r < vdim) bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(v + (size_t)(t0 + i) * in_stride + (size_t)h * vdim + r)), vf);
        if (act) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            qf[e] = silu_f(qf[e]);
            kf[e] = silu_f(kf[e]);
            vf[e] = silu_f(vf[e]);
          }
        }
      }
      uint4 qo, ko, vo;
      qo.x = rc_pack(__float2bfloat16_rn(qf[0]), __float2bfloat16_rn(qf[1])); qo.y = rc_pack(__float2bfloat16_rn(qf[2]), __float2bfloat16_rn(qf[3]));
      qo.z = rc_pack(__float2bfloat16_rn(qf[4]), __float2bfloat16_rn(qf[5])); qo.w = rc_pack(__float2bfloat16_rn(qf[6]), __float2bfloat16_rn(qf[7]));
      ko.x = rc_pack(__float2bfloat16_rn(kf[0]), __float2bfloat16_rn(kf[1])); ko.y = rc_pack(__float2bfloat16_rn(kf[2]), __float2bfloat16_rn(kf[3]));
      ko.z = rc_pack(__float2bfloat16_rn(kf[4]), __float2bfloat16_rn(kf[5])); ko.w = rc_pack(__float2bfloat16_rn(kf[6]), __float2bfloat16_rn(kf[7]));
      vo.x = rc_pack(__float2bfloat16_rn(vf[0]), __float2bfloat16_rn(vf[1])); vo.y = rc_pack(__float2bfloat16_rn(vf[2]), __float2bfloat16_rn(vf[3]));
      vo.z = rc_pack(__float2bfloat16_rn(vf[4]), __float2bfloat16_rn(vf[5])); vo.w = rc_pack(__float2bfloat16_rn(vf[6]), __float2bfloat16_rn(vf[7]));
      *reinterpret_cast<uint4*>(q_s + i * STRIDE + r) = qo;
      *reinterpret_cast<uint4*>(k_s + i * STRIDE + r) = ko;
      *reinterpret_cast<uint4*>(v_s + i * STRIDE + r) = vo;
    }
  } else {
#pragma unroll 4
    for (int idx = tid; idx < DC * HD; idx += 128) {
      const int i = idx / HD, r = idx - i * HD;
      float qv = 0.f, kv = 0.f, vv = 0.f;
      if (i < n) {
        if (r < dim) {
          const size_t at = (size_t)(t0 + i) * in_stride + (size_t)h * dim + r;
          qv = __bfloat162float(q[at]);
          kv = __bfloat162float(k[at]);
          if (act) {
            qv = silu_f(qv);
            kv = silu_f(kv);
          }
        }
        if (r < vdim) {
          vv = __bfloat162float(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + r]);
          if (act) vv = silu_f(vv);
        }
      }
      q_s[i * STRIDE + r] = __float2bfloat16_rn(qv);
      k_s[i * STRIDE + r] = __float2bfloat16_rn(kv);
      v_s[i * STRIDE + r] = __float2bfloat16_rn(vv);
    }
  }
  for (int idx = tid; idx < 3 * DC * 8; idx += 128) q_s[(idx >> 3) * STRIDE + HD + (idx & 7)] = zero;  // the rows' padding
  __syncthreads();

  // ---- the chunk's scores for this warp's 16 tokens against its 64 tokens
  float s_acc[DC / 8][4];
#pragma unroll
  for (int i = 0; i < DC / 8; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    uint32_t a[4];
    rc_ldmatrix_x4(a, q_s + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
    for (int np = 0; np < DC / 16; ++np) {
      uint32_t b[4];
      rc_ldmatrix_x4(b, k_s + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + kk * 16 + 8 * ((lane >> 3) & 1));
      rc_mma_bf16(s_acc[2 * np], a, b[0], b[1]);
      rc_mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
    }
  }
  // ---- decay and mask in 32-bit; each score as two bfloat16 numbers, laid out as the A operand of the next product
  uint32_t p_hi[DC / 16][4], p_lo[DC / 16][4];
  const int row[2] = {warp * 16 + g, warp * 16 + g + 8};
#pragma unroll
  for (int kk = 0; kk < DC / 16; ++kk) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {    // the two groups of 8 keys of this step
#pragma unroll
      for (int r = 0; r < 2; ++r) {           // this thread's two rows
        const int nn = 2 * kk + half;
        bf16 hi[2], lo[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = nn * 8 + 2 * t4 + e;
          const float p = (j <= row[r]) ? s_acc[nn][2 * r + e] * pw[row[r] - j] : 0.f;
          rc_split(p, hi[e], lo[e]);
        }
        p_hi[kk][2 * half + r] = rc_pack(hi[0], hi[1]);
        p_lo[kk][2 * half + r] = rc_pack(lo[0], lo[1]);
      }
    }
  }
  float intra[HD / 8][4], inter[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    intra[i][0] = intra[i][1] = intra[i][2] = intra[i][3] = 0.f;
    inter[i][0] = inter[i][1] = inter[i][2] = inter[i][3] = 0.f;
  }
#pragma unroll
  for (int kk = 0; kk < DC / 16; ++kk) {
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b[4];
      rc_ldmatrix_x4_trans(b, v_s + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
      rc_mma_bf16(intra[2 * dp], p_hi[kk], b[0], b[1]);
      rc_mma_bf16(intra[2 * dp + 1], p_hi[kk], b[2], b[3]);
      rc_mma_bf16(intra[2 * dp], p_lo[kk], b[0], b[1]);
      rc_mma_bf16(intra[2 * dp + 1], p_lo[kk], b[2], b[3]);
    }
  }
  // ---- the queries against the state before the chunk, one bfloat16 half of it at a time in the keys' and values' place
  const float* sp = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vdim;
  bf16* st_s = k_s;  // [HD][STRIDE]: 2 DC rows >= HD
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();  // the keys and values (or the first half) are no longer read
    if ((vdim & 3) == 0) {  // four numbers a load, four loads in flight
#pragma unroll 4
      for (int idx = tid; idx < HD * (HD / 4); idx += 128) {
        const int r = idx / (HD / 4), cc = 4 * (idx - r * (HD / 4));
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < dim && cc < vdim) t = __ldcg(reinterpret_cast<const float4*>(sp + (size_t)r * vdim + cc));
        const float f[4] = {t.x, t.y, t.z, t.w};
        bf16 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          bf16 hi, lo;
          rc_split(f[e], hi, lo);
          o[e] = pass == 0 ? hi : lo;
        }
        uint2 raw;
        raw.x = rc_pack(o[0], o[1]);
        raw.y = rc_pack(o[2], o[3]);
        *reinterpret_cast<uint2*>(st_s + r * STRIDE + cc) = raw;
      }
    } else {
      for (int idx = tid; idx < HD * HD; idx += 128) {
        const int r = idx / HD, cc = idx - r * HD;
        bf16 hi = zero, lo = zero;
        if (r < dim && cc < vdim) rc_split(sp[(size_t)r * vdim + cc], hi, lo);
        st_s[r * STRIDE + cc] = pass == 0 ? hi : lo;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4];
      rc_ldmatrix_x4(a, q_s + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        rc_ldmatrix_x4_trans(b, st_s + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
        rc_mma_bf16(inter[2 * dp], a, b[0], b[1]);
        rc_mma_bf16(inter[2 * dp + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = row[r];
    if (i < n) {
      const float w = pw[i + 1];
      float* o = out + (size_t)(t0 + i) * out_stride + (size_t)h * vdim;
#pragma unroll
      for (int nn = 0; nn < HD / 8; ++nn) {
        const int d = nn * 8 + 2 * t4;
        if (d < vdim) o[d] = intra[nn][2 * r] + w * inter[nn][2 * r];
        if (d + 1 < vdim) o[d + 1] = intra[nn][2 * r + 1] + w * inter[nn][2 * r + 1];
      }
    }
  }
}

// (1) on the tensor cores, for bfloat16 runs with key and value sizes of 33 to 128: U = (K w)^T V over the chunk's tokens, with the
// decay-weighted keys (32-bit) as two bfloat16 halves and the values as bfloat16 after their activation.  A block of four warps
// per (sequence, head, chunk); warp w owns rows HD/4 w .. of U.  The keys lie in shared memory as [token][dim], which is the
// transpose of the product's first operand: `ldmatrix.trans` turns each 8 x 8 piece as it loads it.
template <int HD>
__global__ void __launch_bounds__(128)
decay_chunk_state_mma_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, int in_stride, const float* __restrict__ decay,
                             const int* __restrict__ seq_start, float* __restrict__ scratch, int max_chunks, int H, int dim, int vdim, int act) {
  constexpr int STRIDE = HD + 8;
  constexpr int MT = HD / 64;  // 16-row tiles per warp
  extern __shared__ __align__(16) unsigned char rc_smem[];
  bf16* kh_s = reinterpret_cast<bf16*>(rc_smem);  // [DC][STRIDE] the weighted keys, rounded
  bf16* kl_s = kh_s + DC * STRIDE;                // [DC][STRIDE] what the rounding left
  bf16* v_s = kl_s + DC * STRIDE;                 // [DC][STRIDE]
  __shared__ float pw[DC];
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y;
  const int t0 = seq_start[s] + c * DC;
  const int n = min(DC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const float lam = decay[h];
  if (tid < DC) pw[tid] = powf(lam, (float)tid);
  __syncthreads();
  const bool vec8 = ((dim | vdim | in_stride) & 7) == 0 && ((((uintptr_t)k) | ((uintptr_t)v)) & 15) == 0;
  for (int idx = tid; idx < DC * (HD / 8); idx += 128) {
    const int i = idx / (HD / 8), r = 8 * (idx - i * (HD / 8));
    float kf[8], vf[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) kf[e] = vf[e] = 0.f;
    if (i < n) {
      const size_t row = (size_t)(t0 + i) * in_stride;
      if (vec8) {
        if (r < dim) bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(k + row + (size_t)h * dim + r)), kf);
        if (r < vdim) bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(v + row + (size_t)h * vdim + r)), vf);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (r + e < dim) kf[e] = __bfloat162float(k[row + (size_t)h * dim + r + e]);
          if (r + e < vdim) vf[e] = __bfloat162float(v[row + (size_t)h * vdim + r + e]);
        }
      }
      const float w = pw[n - 1 - i];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        kf[e] = (act ? silu_f(kf[e]) : kf[e]) * w;
        if (act) vf[e] = silu_f(vf[e]);
      }
    }
    bf16 hi[8], lo[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) rc_split(kf[e], hi[e], lo[e]);
    uint4 ho, lo4, vo;
    ho.x = rc_pack(hi[0], hi[1]); ho.y = rc_pack(hi[2], hi[3]); ho.z = rc_pack(hi[4], hi[5]); ho.w = rc_pack(hi[6], hi[7]);
    lo4.x = rc_pack(lo[0], lo[1]); lo4.y = rc_pack(lo[2], lo[3]); lo4.z = rc_pack(lo[4], lo[5]); lo4.w = rc_pack(lo[6], lo[7]);
    vo.x = rc_pack(__float2bfloat16_rn(vf[0]), __float2bfloat16_rn(vf[1])); vo.y = rc_pack(__float2bfloat16_rn(vf[2]), __float2bfloat16_rn(vf[3]));
    vo.z = rc_pack(__float2bfloat16_rn(vf[4]), __float2bfloat16_rn(vf[5])); vo.w = rc_pack(__float2bfloat16_rn(vf[6]), __float2bfloat16_rn(vf[7]));
    *reinterpret_cast<uint4*>(kh_s + i * STRIDE + r) = ho;
    *reinterpret_cast<uint4*>(kl_s + i * STRIDE + r) = lo4;
    *reinterpret_cast<uint4*>(v_s + i * STRIDE + r) = vo;
  }
  __syncthreads();
  float acc[MT][HD / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) acc[mt][i][0] = acc[mt][i][1] = acc[mt][i][2] = acc[mt][i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DC / 16; ++kk) {
    uint32_t a_hi[MT][4], a_lo[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r0 = warp * (HD / 4) + mt * 16;
      const size_t at = (size_t)(kk * 16 + 8 * (lane >> 4) + (lane & 7)) * STRIDE + r0 + 8 * ((lane >> 3) & 1);
      rc_ldmatrix_x4_trans(a_hi[mt], kh_s + at);
      rc_ldmatrix_x4_trans(a_lo[mt], kl_s + at);
    }
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b[4];
      rc_ldmatrix_x4_trans(b, v_s + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        rc_mma_bf16(acc[mt][2 * dp], a_hi[mt], b[0], b[1]);
        rc_mma_bf16(acc[mt][2 * dp + 1], a_hi[mt], b[2], b[3]);
        rc_mma_bf16(acc[mt][2 * dp], a_lo[mt], b[0], b[1]);
        rc_mma_bf16(acc[mt][2 * dp + 1], a_lo[mt], b[2], b[3]);
      }
    }
  }
  float* u = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vdim;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = warp * (HD / 4) + mt * 16 + g + 8 * half;
      if (r < dim) {
#pragma unroll
        for (int nn = 0; nn < HD / 8; ++nn) {
          const int col = nn * 8 + 2 * t4;
          if (col < vdim) u[(size_t)r * vdim + col] = acc[mt][nn][2 * half];
          if (col + 1 < vdim) u[(size_t)r * vdim + col + 1] = acc[mt][nn][2 * half + 1];
        }
      }
    }
  }
}

template <int HD>
static cudaError_t launch_chunk_state_mma(dim3 grid, cudaStream_t stream, const void* k, const void* v, int in_stride, const float* decay,
                                          const int* seq_start, float* scratch, int max_chunks, int H, int dim, int vdim, int act) {
  const size_t smem = (size_t)3 * DC * (HD + 8) * sizeof(bf16);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decay_chunk_state_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  decay_chunk_state_mma_kernel<HD><<<grid, 128, smem, stream>>>((const bf16*)k, (const bf16*)v, in_stride, decay, seq_start, scratch, max_chunks, H,
                                                                dim, vdim, act);
  return cudaGetLastError();
}

template <int HD>
static cudaError_t launch_chunk_out_mma(dim3 grid, cudaStream_t stream, const void* q, const void* k, const void* v, int in_stride,
                                        const float* decay, const int* seq_start, const float* scratch, int max_chunks, float* out,
                                        int out_stride, int H, int dim, int vdim, int act) {
  const size_t smem = (size_t)3 * DC * (HD + 8) * sizeof(bf16);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decay_chunk_out_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  decay_chunk_out_mma_kernel<HD><<<grid, 128, smem, stream>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, in_stride, decay, seq_start, scratch,
                                                              max_chunks, out, out_stride, H, dim, vdim, act);
  return cudaGetLastError();
}

RL_API long long rl_decay_attn_chunked_scratch_floats(int n_seqs, int max_q_len, int H, int dim, int vdim) {
  return (long long)n_seqs * H * ((max_q_len + DC - 1) / DC) * dim * vdim;
}

RL_API int rl_decay_attn_chunked(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* decay, float* state,
                                 const int* slot_ids, const int* seq_start, float* scratch, float* out, int out_stride, int n_seqs,
                                 int max_q_len, int H, int dim, int vdim, int act, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || !scratch)
    RL_REFUSE(1, "decay_attn_chunked: S=%d max_q=%d H=%d dim=%d vdim=%d", n_seqs, max_q_len, H, dim, vdim);
  if (dim > 256) RL_REFUSE(2, "decay_attn_chunked: key size %d exceeds 256", dim);
  const int max_chunks = (max_q_len + DC - 1) / DC, col_tiles = (vdim + DC_COLS - 1) / DC_COLS;
  if (max_chunks > 65535 || col_tiles > 65535) RL_REFUSE(3, "decay_attn_chunked: %d chunks or %d column tiles exceed the grid", max_chunks, col_tiles);
  dim3 grid(n_seqs * H, max_chunks, col_tiles);
  const size_t smem1 = ((size_t)DC * dim + DC * DC_COLS) * sizeof(float);
  const size_t smem3 = ((size_t)2 * DC * (dim + 1) + DC * DC_COLS + DC * (DC + 1) + DC + 1) * sizeof(float);
  const int elems = dim * vdim;
  dim3 grid2(n_seqs * H, (elems + 255) / 256);
#define RL_DAC(T)                                                                                                                     \
  do {                                                                                                                                \
    if (cudaFuncSetAttribute(decay_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1) != cudaSuccess ||  \
        cudaFuncSetAttribute(decay_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3) != cudaSuccess)      \
      RL_REFUSE(4, "decay_attn_chunked: %zu bytes of shared memory refused", smem3);                                                 \
    decay_chunk_state_kernel<T><<<grid, 256, smem1, stream>>>((const T*)k, (const T*)v, in_stride, decay, seq_start, scratch, max_chunks, \
                                                              H, dim, vdim, act);                                                     \
    decay_chunk_scan_kernel<<<grid2, 256, 0, stream>>>(decay, state, slot_ids, seq_start, scratch, max_chunks, H, elems);               \
    decay_chunk_out_kernel<T><<<grid, 256, smem3, stream>>>((const T*)q, (const T*)k, (const T*)v, in_stride, decay, seq_start, scratch,  \
                                                            max_chunks, out, out_stride, H, dim, vdim, act);                          \
  } while (0)
  const int hd = dim > vdim ? dim : vdim;
  if (dtype == RL_BF16 && hd <= 128) {
    // the chunks' additions and the scan as above; the outputs on the tensor cores
    dim3 grid3(n_seqs * H, max_chunks);
    cudaError_t e = cudaSuccess;
    if (hd > 64) {
      e = launch_chunk_state_mma<128>(grid3, stream, k, v, in_stride, decay, seq_start, scratch, max_chunks, H, dim, vdim, act);
    } else if (hd > 32) {
      e = launch_chunk_state_mma<64>(grid3, stream, k, v, in_stride, decay, seq_start, scratch, max_chunks, H, dim, vdim, act);
    } else {
      if (cudaFuncSetAttribute(decay_chunk_state_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1) != cudaSuccess)
        RL_REFUSE(4, "decay_attn_chunked: %zu bytes of shared memory refused", smem1);
      decay_chunk_state_kernel<bf16><<<grid, 256, smem1, stream>>>((const bf16*)k, (const bf16*)v, in_stride, decay, seq_start, scratch, max_chunks,
                                                                   H, dim, vdim, act);
    }
    if (e != cudaSuccess) {
      snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(e));
      return (int)e;
    }
    decay_chunk_scan_kernel<<<grid2, 256, 0, stream>>>(decay, state, slot_ids, seq_start, scratch, max_chunks, H, elems);
    if (hd <= 32) e = launch_chunk_out_mma<32>(grid3, stream, q, k, v, in_stride, decay, seq_start, scratch, max_chunks, out, out_stride, H, dim, vdim, act);
    else if (hd <= 64) e = launch_chunk_out_mma<64>(grid3, stream, q, k, v, in_stride, decay, seq_start, scratch, max_chunks, out, out_stride, H, dim, vdim, act);
    else e = launch_chunk_out_mma<128>(grid3, stream, q, k, v, in_stride, decay, seq_start, scratch, max_chunks, out, out_stride, H, dim, vdim, act);
    if (e != cudaSuccess) {
      snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(e));
      return (int)e;
    }
    return 0;
  }
  if (dtype == RL_BF16) RL_DAC(bf16);
  else if (dtype == RL_F32) RL_DAC(float);
  else RL_REFUSE(5, "decay_attn_chunked: unknown dtype %d", dtype);
#undef RL_DAC
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- norm of a 32-bit row, weight, gate
template <typename T, typename TW>
__global__ void rms_gate_kernel(const float* __restrict__ x, int x_stride, const TW* __restrict__ w, float eps, const T* __restrict__ gate,
                                int gate_stride, float out_scale, T* __restrict__ out, int out_stride, int n) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
#pragma unroll 8
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  const T* g = gate ? gate + (size_t)t * gate_stride : nullptr;
  T* o = out + (size_t)t * out_stride;
#pragma unroll 4
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float y = xr[i] * inv * to_f32(w[i]);
    if (g) y *= logistic(to_f32(g[i]));
    o[i] = from_f32<T>(y * out_scale);
  }
}

RL_API int rl_rms_gate(const float* x, int x_stride, const void* w, int w_dtype, float eps, const void* gate, int gate_stride,
                       float out_scale, void* out, int out_stride, int act_dtype, int n_rows, int n, cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0 || !x || !w || !out) RL_REFUSE(1, "rms_gate: rows=%d n=%d", n_rows, n);
  const int th = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
#define RL_RG(T, TW)                                                                                                               \
  rms_gate_kernel<T, TW><<<n_rows, th, 0, stream>>>(x, x_stride, (const TW*)w, eps, (const T*)gate, gate_stride, out_scale, (T*)out, \
                                                    out_stride, n)
  if (act_dtype == RL_BF16 && w_dtype == RL_F32) RL_RG(bf16, float);
  else if (act_dtype == RL_BF16 && w_dtype == RL_BF16) RL_RG(bf16, bf16);
  else if (act_dtype == RL_F32 && w_dtype == RL_F32) RL_RG(float, float);
  else RL_REFUSE(2, "rms_gate: unsupported dtypes act=%d w=%d", act_dtype, w_dtype);
#undef RL_RG
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- minimal gated recurrent unit
// One thread per (sequence, channel); the sequence's tokens in order, eight at a time so that their loads are in flight together.
#define GRU_AHEAD 8

template <typename T>
__global__ void min_gru_kernel(const T* __restrict__ z, const T* __restrict__ x, const T* __restrict__ g, int in_stride,
                               const float* __restrict__ z_bias, const float* __restrict__ x_bias, float* __restrict__ state,
                               const int* __restrict__ slot_ids, const int* __restrict__ seq_start, float out_scale, T* __restrict__ out,
                               int out_stride, int width) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* st = state + (size_t)slot_ids[s] * width + c;
  float S = *st;
  const float bz = z_bias ? z_bias[c] : 0.f, bx = x_bias ? x_bias[c] : 0.f;
  for (int base = t0; base < t1; base += GRU_AHEAD) {
    float zv[GRU_AHEAD], xv[GRU_AHEAD], gv[GRU_AHEAD];
#pragma unroll
    for (int j = 0; j < GRU_AHEAD; ++j) {
      if (base + j < t1) {
        const size_t at = (size_t)(base + j) * in_stride + c;
        zv[j] = to_f32(z[at]);
        xv[j] = to_f32(x[at]);
        gv[j] = to_f32(g[at]);
      }
    }
#pragma unroll
    for (int j = 0; j < GRU_AHEAD; ++j) {
      if (base + j < t1) {
        const float zz = logistic(zv[j] + bz);
        const float u = xv[j] + bx;
        const float cand = u >= 0.f ? u + 0.5f : logistic(u);
        S = (1.0f - zz) * S + zz * cand;
        out[(size_t)(base + j) * out_stride + c] = from_f32<T>(S * silu_f(gv[j]) * out_scale);
      }
    }
  }
  *st = S;
}

// The same for long prompts: a sequence's tokens are cut into GRU_SEGS stretches, one per warp.  Each warp first runs its stretch
// from a zero state, which gives the stretch as a map S -> A S + B; the maps before a stretch, applied in order to the sequence's
// state, give the state it starts from; a second run through the stretch writes the results.  (The sums come out in another
// order than in the token-by-token kernel, and the order depends on where the stretches fall.)
#define GRU_SEGS 32

template <typename T>
__global__ void __launch_bounds__(32 * GRU_SEGS)
min_gru_seg_kernel(const T* __restrict__ z, const T* __restrict__ x, const T* __restrict__ g, int in_stride, const float* __restrict__ z_bias,
                   const float* __restrict__ x_bias, float* __restrict__ state, const int* __restrict__ slot_ids,
                   const int* __restrict__ seq_start, float out_scale, T* __restrict__ out, int out_stride, int width) {
  __shared__ float A_s[GRU_SEGS][32], B_s[GRU_SEGS][32];
  const int lane = threadIdx.x, w = threadIdx.y;
  const int s = blockIdx.x, c = blockIdx.y * 32 + lane;
  const bool ok = c < width;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  const int seg = (t1 - t0 + GRU_SEGS - 1) / GRU_SEGS;
  const int a = min(t1, t0 + w * seg), b = min(t1, a + seg);
  const float bz = (ok && z_bias) ? z_bias[c] : 0.f, bx = (ok && x_bias) ? x_bias[c] : 0.f;
  float A = 1.f, B = 0.f;
  if (ok) {
    for (int base = a; base < b; base += 8) {
      float zv[8], xv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (base + j < b) {
          const size_t at = (size_t)(base + j) * in_stride + c;
          zv[j] = to_f32(z[at]);
          xv[j] = to_f32(x[at]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (base + j < b) {
          const float zz = logistic(zv[j] + bz);
          const float u = xv[j] + bx;
          const float cand = u >= 0.f ? u + 0.5f : logistic(u);
          B = (1.0f - zz) * B + zz * cand;
          A *= 1.0f - zz;
        }
      }
    }
  }
  A_s[w][lane] = A;
  B_s[w][lane] = B;
  __syncthreads();
  if (!ok) return;
  float* st = state + (size_t)slot_ids[s] * width + c;
  float S = *st;
  for (int j = 0; j < w; ++j) S = A_s[j][lane] * S + B_s[j][lane];
  for (int base = a; base < b; base += 8) {
    float zv[8], xv[8], gv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (base + j < b) {
        const size_t at = (size_t)(base + j) * in_stride + c;
        zv[j] = to_f32(z[at]);
        xv[j] = to_f32(x[at]);
        gv[j] = to_f32(g[at]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (base + j < b) {
        const float zz = logistic(zv[j] + bz);
        const float u = xv[j] + bx;
        const float cand = u >= 0.f ? u + 0.5f : logistic(u);
        S = (1.0f - zz) * S + zz * cand;
        out[(size_t)(base + j) * out_stride + c] = from_f32<T>(S * silu_f(gv[j]) * out_scale);
      }
    }
  }
  if (w == GRU_SEGS - 1) *st = S;
}

// max_q_len: the most tokens that a sequence of the step brings if the caller allows the stretch-wise kernel for long sequences
// (results then depend on how a sequence was cut into steps, within rounding); 0: token by token, the same bits for every cut.
RL_API int rl_min_gru(const void* z, const void* x, const void* g, int dtype, int in_stride, const float* z_bias, const float* x_bias,
                      float* state, const int* slot_ids, const int* seq_start, float out_scale, void* out, int out_stride, int n_seqs,
                      int width, int max_q_len, cudaStream_t stream) {
  if (n_seqs <= 0 || width <= 0 || !z || !x || !g || !state || !out) RL_REFUSE(1, "min_gru: S=%d width=%d", n_seqs, width);
  if (max_q_len >= 8 * GRU_SEGS) {
    dim3 grid(n_seqs, (width + 31) / 32), block(32, GRU_SEGS);
    if (dtype == RL_BF16)
      min_gru_seg_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)z, (const bf16*)x, (const bf16*)g, in_stride, z_bias, x_bias, state,
                                                           slot_ids, seq_start, out_scale, (bf16*)out, out_stride, width);
    else if (dtype == RL_F32)
      min_gru_seg_kernel<float><<<grid, block, 0, stream>>>((const float*)z, (const float*)x, (const float*)g, in_stride, z_bias, x_bias,
                                                            state, slot_ids, seq_start, out_scale, (float*)out, out_stride, width);
    else
      RL_REFUSE(2, "min_gru: unknown dtype %d", dtype);
    RL_LAUNCH_RESULT();
  }
  const int th = width >= 128 ? 128 : ((width + 31) / 32) * 32;
  dim3 grid(n_seqs, (width + th - 1) / th);
  if (dtype == RL_BF16)
    min_gru_kernel<bf16><<<grid, th, 0, stream>>>((const bf16*)z, (const bf16*)x, (const bf16*)g, in_stride, z_bias, x_bias, state, slot_ids,
                                                  seq_start, out_scale, (bf16*)out, out_stride, width);
  else if (dtype == RL_F32)
    min_gru_kernel<float><<<grid, th, 0, stream>>>((const float*)z, (const float*)x, (const float*)g, in_stride, z_bias, x_bias, state,
                                                   slot_ids, seq_start, out_scale, (float*)out, out_stride, width);
  else
    RL_REFUSE(2, "min_gru: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- element-wise activation
#define RL_ACT_RELU2 1

template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, T* __restrict__ y, long long total, int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = fmaxf(to_f32(x[i]), 0.f);
  y[i] = from_f32<T>(v * v);
}

RL_API int rl_unary_act(const void* x, void* y, int dtype, long long total, int kind, cudaStream_t stream) {
  if (total <= 0) RL_REFUSE(1, "unary_act: nothing to do");
  if (kind != RL_ACT_RELU2) RL_REFUSE(2, "unary_act: unknown activation %d", kind);
  const long long blocks = (total + 255) / 256;
  if (dtype == RL_BF16) unary_act_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>((const bf16*)x, (bf16*)y, total, kind);
  else if (dtype == RL_F32) unary_act_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((const float*)x, (float*)y, total, kind);
  else RL_REFUSE(3, "unary_act: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}
