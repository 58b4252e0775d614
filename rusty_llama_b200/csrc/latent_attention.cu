// Latent attention: every head's keys and values are linear maps of one small vector per position
// (the latent c, `rank` numbers) plus one rotated key part shared by all heads (`rot` numbers), and only
// those rank + rot numbers are cached.  The kernels here work on the cached row directly:
//
//   score(t, h, j) = ( q_lat[t,h] . c_j  +  q_rot[t,h] . kr_j ) * scale      q_lat[t,h] = W_uk[h]^T q_plain[t,h]
//   o_lat[t,h]     = sum_j p(t,h,j) c_j                                       head output = W_uv[h] o_lat[t,h]
//
// which is the same arithmetic as expanding every cached position into per-head keys and values, with the
// two small per-head maps moved to the query and to the result.  All heads then read one row per key: the
// cache is read once per query token, not once per head.
//
//   latent_prep    per token: RMS-norm of the latent, rotation of the shared key part, both stored into the
//                  token's place in the paged cache; rotation of every head's rotated query part into the
//                  tail of the head's row of q_cat[T, H, rank + rot]
//   head_linear    out[t,h,:] = W[h] x[t,h,:], one small product per head (the two absorbed maps), optionally
//                  times sigmoid(gate[t,h,:]) (the mixer's output gate)
//   latent_attn    softmax attention with a sink over the cached rows; any sizes, both element types, keys
//                  always taken in the same groups of 32 from position 0, so the bits of a result do not
//                  depend on how a sequence was cut into steps or on what else is in the batch
//
// Softmax with a sink: the denominator has one more term exp(sink[h]) that has no key and no value; it is
// the start value of the running maximum and sum (m = sink, l = 1, o = 0).
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

// ---------------------------------------------------------------- norm, rotation, cache write
// Pair i of a rotated part, dimensions (2i, 2i+1), turns by pos * freq[i]; cos and sin are multiplied by
// `mag`; pairs from n_pairs on pass unchanged.  Everything in 32-bit, rounded once when stored.
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ kv, int ldkv,
                                   const float* __restrict__ norm_w, float eps, const float* __restrict__ freq,
                                   int n_pairs, float mag, const int* __restrict__ tok_pos,
                                   const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                   int table_width, T* __restrict__ pages, int page_size, T* __restrict__ q_cat,
                                   int H, int dim, int rot, int rank) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int Dk = rank + rot;
  if (kv != nullptr) {
    const T* row = kv + (size_t)t * ldkv;
    const int page = block_table[(size_t)tok_seq[t] * table_width + pos / page_size];
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * Dk;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float v = to_f32(row[i]);
      ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(row[i]) * inv * norm_w[i]);
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
      float u = to_f32(row[rank + 2 * i]), v = to_f32(row[rank + 2 * i + 1]);
      if (i < n_pairs) {
        float s, c;
        sincosf((float)pos * freq[i], &s, &c);
        s *= mag;
        c *= mag;
        const float a = u * c - v * s, b = v * c + u * s;
        u = a;
        v = b;
      }
      dst[rank + 2 * i] = from_f32<T>(u);
      dst[rank + 2 * i + 1] = from_f32<T>(v);
    }
    if ((rot & 1) && threadIdx.x == 0) dst[rank + rot - 1] = row[rank + rot - 1];
  }
  const int half = rot / 2;
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const T* src = q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim;
    float u = to_f32(src[2 * i]), v = to_f32(src[2 * i + 1]);
    if (i < n_pairs) {
      float s, c;
      sincosf((float)pos * freq[i], &s, &c);
      s *= mag;
      c *= mag;
      const float a = u * c - v * s, b = v * c + u * s;
      u = a;
      v = b;
    }
    T* dst = q_cat + ((size_t)t * H + h) * Dk + rank;
    dst[2 * i] = from_f32<T>(u);
    dst[2 * i + 1] = from_f32<T>(v);
  }
  if (rot & 1)
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      q_cat[((size_t)t * H + h) * Dk + rank + rot - 1] = q[(size_t)t * ldq + (size_t)h * (dim + rot) + dim + rot - 1];
}

RL_API int rl_latent_prep(const void* q, int ldq, const void* kv, int ldkv, int dtype, const float* norm_w, float eps,
                          const float* freq, int n_pairs, float mag, const int* tok_pos, const int* tok_seq,
                          const int* block_table, int table_width, void* pages, int page_size, void* q_cat,
                          int n_tokens, int H, int dim, int rot, int rank, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || dim < 0 || rot < 0 || rank <= 0 || page_size <= 0)
    RL_REFUSE(1, "latent_prep: T=%d H=%d dim=%d rot=%d rank=%d page=%d", n_tokens, H, dim, rot, rank, page_size);
  if (2 * n_pairs > rot) RL_REFUSE(2, "latent_prep: %d rotated pairs do not fit %d dimensions", n_pairs, rot);
  if (kv != nullptr && (pages == nullptr || block_table == nullptr || norm_w == nullptr))
    RL_REFUSE(3, "latent_prep: a latent row to store, but no pages, page table or norm weight");
  if (dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch<false>(latent_prep_kernel<bf16>, n_tokens, 128, 0, stream, (const bf16*)q, ldq, (const bf16*)kv, ldkv,
                              norm_w, eps, freq, n_pairs, mag, tok_pos, tok_seq, block_table, table_width, (bf16*)pages,
                              page_size, (bf16*)q_cat, H, dim, rot, rank));
  else if (dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(latent_prep_kernel<float>, n_tokens, 128, 0, stream, (const float*)q, ldq, (const float*)kv,
                              ldkv, norm_w, eps, freq, n_pairs, mag, tok_pos, tok_seq, block_table, table_width,
                              (float*)pages, page_size, (float*)q_cat, H, dim, rot, rank));
  else
    RL_REFUSE(4, "latent_prep: unknown dtype %d", dtype);
  return 0;
}

// ---------------------------------------------------------------- one small product per head
// out[t, h, n] = sum_k x[t, h, k] * w[h, n, k]   (k ascending, one running 32-bit sum per output),
// optionally times sigmoid(gate[t, h, n]) computed in 32-bit.  x, out and gate are addressed as
// base + t * ld + h * head_stride + i; w as base + h * w_head + n * ldw + k, so that a transposed map
// (w[h, k, n] stored, ldw = 1) is the same kernel.
#define HL_TM 64
#define HL_TN 64
#define HL_TK 16

template <typename T, bool GATE>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, int ldx, int xh, const T* __restrict__ w, long long w_head, int w_n, int w_k,
                   T* __restrict__ out, int ldo, int oh, const T* __restrict__ gate, int ldg, int gh, int M, int N, int K) {
  __shared__ float xs[HL_TK][HL_TM + 4];
  __shared__ float ws[HL_TK][HL_TN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, h = blockIdx.z;
  const int m0 = blockIdx.y * HL_TM, n0 = blockIdx.x * HL_TN;
  const int ty = tid / 16, tx = tid % 16;
  x += (size_t)h * xh;
  w += (size_t)h * w_head;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HL_TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx / HL_TK, c = idx % HL_TK;
      const int k = k0 + c;
      xs[c][r] = (m0 + r < M && k < K) ? to_f32(x[(size_t)(m0 + r) * ldx + k]) : 0.f;
      ws[c][r] = (n0 + r < N && k < K) ? to_f32(w[(size_t)(n0 + r) * w_n + (size_t)k * w_k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < HL_TK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (GATE) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)m * ldg + (size_t)h * gh + n])));
      out[(size_t)m * ldo + (size_t)h * oh + n] = from_f32<T>(v);
    }
  }
}

RL_API int rl_head_linear(const void* x, int ldx, int xh, const void* w, long long w_head, int w_n, int w_k, void* out,
                          int ldo, int oh, const void* gate, int ldg, int gh, int dtype, int M, int H, int N, int K,
                          cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "head_linear: M=%d H=%d N=%d K=%d", M, H, N, K);
  const int gy = (M + HL_TM - 1) / HL_TM;
  if (gy > 65535 || H > 65535) RL_REFUSE(2, "head_linear: %d rows or %d heads exceed the grid", M, H);
  dim3 grid((N + HL_TN - 1) / HL_TN, gy, H);
#define RL_HL(T, G)                                                                                                    \
  RL_LAUNCH_CHECK(rl_launch<false>(head_linear_kernel<T, G>, grid, 256, 0, stream, (const T*)x, ldx, xh, (const T*)w, w_head, \
                            w_n, w_k, (T*)out, ldo, oh, (const T*)gate, ldg, gh, M, N, K))
  if (dtype == RL_BF16 && gate) RL_HL(bf16, true);
  else if (dtype == RL_BF16) RL_HL(bf16, false);
  else if (dtype == RL_F32 && gate) RL_HL(float, true);
  else if (dtype == RL_F32) RL_HL(float, false);
  else RL_REFUSE(3, "head_linear: unknown dtype %d", dtype);
#undef RL_HL
  return 0;
}

// ---------------------------------------------------------------- attention over the cached rows, the plain way
// One warp per (token, head).  A cached row is [rank latent | rot shared key part]; the query row has the same
// layout; the result is the probability-weighted sum of the latent parts.  Keys in groups of 32 from position 0
// (or from the first key inside `window`, if one is given), online softmax that starts from the sink.
#define LA_MAX_PER_LANE 32  // latent sizes up to 1024

template <typename T>
__global__ void latent_attn_kernel(const T* __restrict__ q_cat, const T* __restrict__ pages,
                                   const int* __restrict__ block_table, int table_width,
                                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                   const float* __restrict__ sink, T* __restrict__ out, int H, int rank, int rot,
                                   int page_size, int window, float scale) {
  extern __shared__ float q_s[];  // rank + rot floats
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x;
  const int t = blockIdx.x, h = blockIdx.y;
  const int Dk = rank + rot;
  const int pos = tok_pos[t];
  const int* table = block_table + (size_t)tok_seq[t] * table_width;
  const T* qh = q_cat + ((size_t)t * H + h) * Dk;
  for (int i = lane; i < Dk; i += 32) q_s[i] = to_f32(qh[i]);
  __syncwarp();
  const int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
  float acc[LA_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < LA_MAX_PER_LANE; ++i) acc[i] = 0.f;
  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float s = -INFINITY;
    if (valid) {
      const T* kr = pages + ((size_t)table[key / page_size] * page_size + key % page_size) * Dk;
      float dot = 0.f;
      for (int i = 0; i < Dk; ++i) dot += q_s[i] * to_f32(kr[i]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LA_MAX_PER_LANE; ++i) acc[i] *= alpha;
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const T* vr = pages + ((size_t)table[kj / page_size] * page_size + kj % page_size) * Dk;
#pragma unroll
      for (int i = 0; i < LA_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] += pj * to_f32(vr[d]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + ((size_t)t * H + h) * rank;
#pragma unroll
  for (int i = 0; i < LA_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) o[d] = from_f32<T>(acc[i] * inv);
  }
}

RL_API int rl_latent_attn(const void* q_cat, const void* pages, int dtype, const int* block_table, int table_width,
                          const int* tok_seq, const int* tok_pos, const float* sink, void* out, int n_tokens, int H,
                          int rank, int rot, int page_size, int window, float scale, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || rank <= 0 || rot < 0 || page_size <= 0)
    RL_REFUSE(1, "latent_attn: T=%d H=%d rank=%d rot=%d page=%d", n_tokens, H, rank, rot, page_size);
  if (rank > 32 * LA_MAX_PER_LANE) RL_REFUSE(2, "latent_attn: latent size %d exceeds %d", rank, 32 * LA_MAX_PER_LANE);
  if (H > 65535) RL_REFUSE(3, "latent_attn: %d heads exceed 65535", H);
  if (window < 0) RL_REFUSE(4, "latent_attn: negative window");
  dim3 grid(n_tokens, H);
  const size_t smem = (size_t)(rank + rot) * sizeof(float);
  if (dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch<false>(latent_attn_kernel<bf16>, grid, 32, smem, stream, (const bf16*)q_cat, (const bf16*)pages,
                              block_table, table_width, tok_seq, tok_pos, sink, (bf16*)out, H, rank, rot, page_size,
                              window, scale));
  else if (dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(latent_attn_kernel<float>, grid, 32, smem, stream, (const float*)q_cat, (const float*)pages,
                              block_table, table_width, tok_seq, tok_pos, sink, (float*)out, H, rank, rot, page_size,
                              window, scale));
  else
    RL_REFUSE(5, "latent_attn: unknown dtype %d", dtype);
  return 0;
}
