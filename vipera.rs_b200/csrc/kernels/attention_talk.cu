// Causal grouped-query softmax attention over the paged cache whose head weights are mixed by a
// matrix before they meet the values ("talking heads" behind the softmax):
//
//   p_g(i, j) = softmax_j((q_g(i) . k_kv(g)(j)) * scale)          for every query head g
//   w_h(i, j) = sum_g M[h, g] p_g(i, j)
//   o_h(i)    = sum_j w_h(i, j) v_kv(h)(j)
//
// Head h applies its mixed weights to the values of its own KV head.  The mix needs the
// normalised weights of all heads at one (query, key), so a block owns a token and all its heads,
// and runs over the keys twice: the first pass finds every head's maximum and sum, the second
// forms p for a tile of 32 keys per head in shared memory, mixes, and folds the values.  Scores,
// weights, the mix and the accumulation are 32-bit.  Keys are found through the block table.
//
// The same kernel serves portions of prompts and single tokens, both element types, head sizes up
// to 256 and up to 64 heads.  A warp owns HPW heads (heads warp, warp + kTalkWarps, ...).
#include "common.cuh"

constexpr int kTalkWarps = 8;
constexpr int kTalkMaxDim = 256;
constexpr int kTalkMaxHeads = 64;

template <typename T>
__device__ __forceinline__ float talk_dot(const float* __restrict__ q, const T* __restrict__ row, int d) {
  float sum = 0.0f;
  for (int i = 0; i < d; ++i) sum = fmaf(q[i], to_float<T>(row[i]), sum);
  return sum;
}

template <typename T, int HPW>
__global__ void __launch_bounds__(kTalkWarps * 32)
attention_talk_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, const float* __restrict__ mix, const int* __restrict__ token_seq,
                      const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
                      int page_size, int num_heads, int num_kv_heads, int head_dim, int value_dim, float scale,
                      float out_scale) {
  extern __shared__ float shared[];
  float* q_s = shared;                                   // [heads][head_dim]
  float* mix_s = q_s + num_heads * head_dim;             // [heads][heads]
  float* p_s = mix_s + num_heads * num_heads;            // [heads][32]
  float* max_s = p_s + num_heads * 32;                   // [heads]
  float* inv_s = max_s + num_heads;                      // [heads]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < num_heads * num_heads; i += blockDim.x) mix_s[i] = mix[i];
  pdl_wait();
  const int t = blockIdx.x;
  const int group = num_heads / num_kv_heads;
  const int position = positions[t];
  const int* table = block_table + static_cast<size_t>(token_seq[t]) * table_width;
  const T* q_row = q + static_cast<size_t>(t) * num_heads * head_dim;
  for (int i = threadIdx.x; i < num_heads * head_dim; i += blockDim.x) q_s[i] = to_float<T>(q_row[i]);
  __syncthreads();
  const size_t k_stride = static_cast<size_t>(num_kv_heads) * head_dim;
  const size_t v_stride = static_cast<size_t>(num_kv_heads) * value_dim;

  // pass 1: maximum and sum of every head this warp owns
#pragma unroll
  for (int s = 0; s < HPW; ++s) {
    const int g = warp + s * kTalkWarps;
    if (g >= num_heads) break;
    const int kv = g / group;
    float running_max = -INFINITY, running_sum = 0.0f;
    for (int base = 0; base <= position; base += 32) {
      const int j = base + lane;
      float score = -INFINITY;
      if (j <= position) {
        const int page = table[j / page_size];
        const T* k_row = k_pool + (static_cast<size_t>(page) * page_size + j % page_size) * k_stride +
                         static_cast<size_t>(kv) * head_dim;
        score = talk_dot<T>(q_s + g * head_dim, k_row, head_dim) * scale;
      }
      const float new_max = fmaxf(running_max, warp_max(score));
      const float weight = j <= position ? expf(score - new_max) : 0.0f;
      running_sum = running_sum * expf(running_max - new_max) + warp_sum(weight);
      running_max = new_max;
    }
    if (lane == 0) {
      max_s[g] = running_max;
      inv_s[g] = 1.0f / running_sum;
    }
  }
  __syncthreads();

  // pass 2: normalised weights of a tile of keys for all heads, mixed, folded into the values
  float acc[HPW][kTalkMaxDim / 32];
#pragma unroll
  for (int s = 0; s < HPW; ++s)
#pragma unroll
    for (int i = 0; i < kTalkMaxDim / 32; ++i) acc[s][i] = 0.0f;
  for (int base = 0; base <= position; base += 32) {
    const int j = base + lane;
    const bool valid = j <= position;
    size_t at = 0;
    if (valid) at = static_cast<size_t>(table[j / page_size]) * page_size + j % page_size;
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
      const int g = warp + s * kTalkWarps;
      if (g >= num_heads) break;
      float p = 0.0f;
      if (valid) {
        const T* k_row = k_pool + at * k_stride + static_cast<size_t>(g / group) * head_dim;
        p = expf(talk_dot<T>(q_s + g * head_dim, k_row, head_dim) * scale - max_s[g]) * inv_s[g];
      }
      p_s[g * 32 + lane] = p;
    }
    __syncthreads();
    const int count = min(32, position - base + 1);
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
      const int h = warp + s * kTalkWarps;
      if (h >= num_heads) break;
      float weight = 0.0f;
      for (int g = 0; g < num_heads; ++g) weight = fmaf(mix_s[h * num_heads + g], p_s[g * 32 + lane], weight);
      const int kv = h / group;
      for (int jj = 0; jj < count; ++jj) {
        const float w = __shfl_sync(0xffffffffu, weight, jj);
        const size_t row = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(at), jj);
        const T* v_row = v_pool + row * v_stride + static_cast<size_t>(kv) * value_dim;
#pragma unroll
        for (int i = 0; i < kTalkMaxDim / 32; ++i) {
          const int e = lane + 32 * i;
          if (e < value_dim) acc[s][i] = fmaf(w, to_float<T>(v_row[e]), acc[s][i]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int s = 0; s < HPW; ++s) {
    const int h = warp + s * kTalkWarps;
    if (h >= num_heads) break;
    T* out_row = out + (static_cast<size_t>(t) * num_heads + h) * value_dim;
#pragma unroll
    for (int i = 0; i < kTalkMaxDim / 32; ++i) {
      const int e = lane + 32 * i;
      if (e < value_dim) out_row[e] = from_float<T>(acc[s][i] * out_scale);
    }
  }
}

template <typename T>
static int launch_talk(int hpw, dim3 grid, size_t shared_bytes, cudaStream_t s, const void* q, void* out, const void* k_pool,
                       const void* v_pool, const float* mix, const int* token_seq, const int* positions,
                       const int* block_table, int table_width, int page_size, int num_heads, int num_kv_heads,
                       int head_dim, int value_dim, float scale, float out_scale) {
#define TALK_CASE(N)                                                                                             \
  {                                                                                                              \
    if (shared_bytes > 48 * 1024) {                                                                              \
      cudaError_t e = cudaFuncSetAttribute(attention_talk_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           static_cast<int>(shared_bytes));                                      \
      if (e != cudaSuccess) return static_cast<int>(e);                                                          \
    }                                                                                                            \
    return vipera_launch(attention_talk_kernel<T, N>, grid, kTalkWarps * 32, shared_bytes, s,                    \
                         static_cast<const T*>(q), static_cast<T*>(out), static_cast<const T*>(k_pool),          \
                         static_cast<const T*>(v_pool), mix, token_seq, positions, block_table, table_width,     \
                         page_size, num_heads, num_kv_heads, head_dim, value_dim, scale, out_scale);             \
  }
  if (hpw <= 1) TALK_CASE(1)
  if (hpw <= 2) TALK_CASE(2)
  if (hpw <= 4) TALK_CASE(4)
  TALK_CASE(8)
#undef TALK_CASE
}

// q [tokens, heads, d], out [tokens, heads, value_dim], mix [heads, heads] 32-bit (row h holds the
// weights of head h's mix); pools and tables as in the general attention kernel.
VIPERA_API int vipera_attention_talk(const void* q, void* out, int dtype, const void* k_pool, const void* v_pool,
                                     const float* mix, const int* token_seq, const int* positions,
                                     const int* block_table, int table_width, int page_size, int num_tokens,
                                     int num_heads, int num_kv_heads, int head_dim, int value_dim, float scale,
                                     float out_scale, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (head_dim <= 0 || head_dim > kTalkMaxDim || value_dim <= 0 || value_dim > kTalkMaxDim) return VIPERA_BAD_SHAPE;
  if (num_heads <= 0 || num_heads > kTalkMaxHeads || num_kv_heads <= 0 || num_heads % num_kv_heads) return VIPERA_BAD_SHAPE;
  if (page_size <= 0 || table_width <= 0 || !mix) return VIPERA_BAD_ARGUMENT;
  const size_t shared_bytes = sizeof(float) * (static_cast<size_t>(num_heads) * head_dim + num_heads * num_heads +
                                               num_heads * 32 + 2 * num_heads);
  if (shared_bytes > 200 * 1024) return VIPERA_BAD_SHAPE;
  const int hpw = (num_heads + kTalkWarps - 1) / kTalkWarps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tokens);
  if (dtype == VIPERA_F32)
    return launch_talk<float>(hpw, grid, shared_bytes, s, q, out, k_pool, v_pool, mix, token_seq, positions, block_table,
                              table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim, scale, out_scale);
  if (dtype == VIPERA_BF16)
    return launch_talk<__nv_bfloat16>(hpw, grid, shared_bytes, s, q, out, k_pool, v_pool, mix, token_seq, positions,
                                      block_table, table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim,
                                      scale, out_scale);
  return VIPERA_BAD_DTYPE;
}
