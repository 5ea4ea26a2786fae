// Causal grouped-query softmax attention over the paged cache whose head weights are mixed by a
// matrix before they meet the values ("talking heads" behind the softmax):
//
//   p_g(i, j) = softmax_j((q_g(i) . k_kv(g)(j)) * scale)          for every query head g
//   w_h(i, j) = sum_g M[h, g] p_g(i, j)
//   o_h(i)    = sum_j w_h(i, j) v_kv(h)(j)
//
// Head h applies its mixed weights to the values of its own KV head.  The mix needs the
// normalised weights of all heads at one (query, key), so a block owns a token and all its heads,
// and the keys are run over twice, by two kernels: the first finds every head's maximum and sum,
// the second forms p for a tile of 32 keys per head in shared memory, mixes, and folds the values.
// The keys are cut into splits (a block a token and a split), so that a step of few tokens with
// long histories fills the GPU; a third kernel then adds the splits' partial outputs in order.
// Scores, weights, the mix and the accumulation are 32-bit.  Keys are found through the block table.
//
// The same kernel serves portions of prompts and single tokens, both element types, head sizes up
// to 256 and up to 64 heads.  A warp owns HPW heads (heads warp, warp + kTalkWarps, ...).
#include "common.cuh"

constexpr int kTalkWarps = 8;
constexpr int kTalkMaxDim = 256;
constexpr int kTalkMaxHeads = 64;

// q . row with 16-byte loads of the row where its size allows them (rows then start on 16 bytes).
template <typename T>
__device__ __forceinline__ float talk_dot(const float* __restrict__ q, const T* __restrict__ row, int d);

template <>
__device__ __forceinline__ float talk_dot<float>(const float* __restrict__ q, const float* __restrict__ row, int d) {
  float sum = 0.0f;
  if (d & 3) {
    for (int i = 0; i < d; ++i) sum = fmaf(q[i], row[i], sum);
    return sum;
  }
  const float4* r4 = reinterpret_cast<const float4*>(row);
  const float4* q4 = reinterpret_cast<const float4*>(q);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = r4[i], w = q4[i];
    sum = fmaf(w.x, v.x, sum);
    sum = fmaf(w.y, v.y, sum);
    sum = fmaf(w.z, v.z, sum);
    sum = fmaf(w.w, v.w, sum);
  }
  return sum;
}

template <>
__device__ __forceinline__ float talk_dot<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row,
                                                         int d) {
  float sum = 0.0f;
  if (d & 7) {
    for (int i = 0; i < d; ++i) sum = fmaf(q[i], __bfloat162float(row[i]), sum);
    return sum;
  }
  const uint4* r8 = reinterpret_cast<const uint4*>(row);
  const float4* q4 = reinterpret_cast<const float4*>(q);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 raw = r8[i];
    const float4 a = q4[2 * i], b = q4[2 * i + 1];
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 f0 = __bfloat1622float2(pairs[0]), f1 = __bfloat1622float2(pairs[1]);
    const float2 f2 = __bfloat1622float2(pairs[2]), f3 = __bfloat1622float2(pairs[3]);
    sum = fmaf(a.x, f0.x, sum);
    sum = fmaf(a.y, f0.y, sum);
    sum = fmaf(a.z, f1.x, sum);
    sum = fmaf(a.w, f1.y, sum);
    sum = fmaf(b.x, f2.x, sum);
    sum = fmaf(b.y, f2.y, sum);
    sum = fmaf(b.z, f3.x, sum);
    sum = fmaf(b.w, f3.y, sum);
  }
  return sum;
}

// Shared memory of both kernels: q [heads][d], the mix [heads][heads], a tile of weights
// [heads][32], and per head the maximum and the inverse sum.
struct TalkShared {
  float *q, *mix, *p, *max, *inv;
  __device__ TalkShared(float* base, int heads, int d) {
    q = base;
    mix = q + heads * d;
    p = mix + heads * heads;
    max = p + heads * 32;
    inv = max + heads;
  }
};

// Pass 1: every head's maximum and sum over the keys of one split.  grid (token, split).
template <typename T, int HPW>
__global__ void __launch_bounds__(kTalkWarps * 32)
talk_stats_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const int* __restrict__ token_seq,
                  const int* __restrict__ positions, const int* __restrict__ block_table, int table_width, int page_size,
                  int num_heads, int num_kv_heads, int head_dim, float scale, int split_keys, int num_splits,
                  float* __restrict__ stats) {
  extern __shared__ __align__(16) float shared[];
  TalkShared sh(shared, num_heads, head_dim);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int t = blockIdx.x, split = blockIdx.y;
  const int group = num_heads / num_kv_heads;
  const int position = positions[t];
  const int begin = split * split_keys, last = min(begin + split_keys - 1, position);
  if (begin > position) return;   // nobody reads the statistics of a split without keys
  const int* table = block_table + static_cast<size_t>(token_seq[t]) * table_width;
  const T* q_row = q + static_cast<size_t>(t) * num_heads * head_dim;
  for (int i = threadIdx.x; i < num_heads * head_dim; i += blockDim.x) sh.q[i] = to_float<T>(q_row[i]);
  __syncthreads();
  const size_t k_stride = static_cast<size_t>(num_kv_heads) * head_dim;
#pragma unroll
  for (int s = 0; s < HPW; ++s) {
    const int g = warp + s * kTalkWarps;
    if (g >= num_heads) break;
    const int kv = g / group;
    float running_max = -INFINITY, running_sum = 0.0f;
    for (int base = begin; base <= last; base += 32) {
      const int j = base + lane;
      float score = -INFINITY;
      if (j <= last) {
        const int page = table[j / page_size];
        const T* k_row = k_pool + (static_cast<size_t>(page) * page_size + j % page_size) * k_stride +
                         static_cast<size_t>(kv) * head_dim;
        score = talk_dot<T>(sh.q + g * head_dim, k_row, head_dim) * scale;
      }
      const float new_max = fmaxf(running_max, warp_max(score));
      const float weight = j <= last ? expf(score - new_max) : 0.0f;
      running_sum = running_sum * expf(running_max - new_max) + warp_sum(weight);
      running_max = new_max;
    }
    if (lane == 0) {
      float* cell = stats + ((static_cast<size_t>(t) * num_splits + split) * num_heads + g) * 2;
      cell[0] = running_max;
      cell[1] = running_sum;
    }
  }
}

// Pass 2: the splits' statistics joined (every block does that for itself, in a fixed order), then
// the normalised weights of a tile of keys for all heads, mixed, folded into the values of this
// split's keys.  With one split the result goes to `out`, else to `partial` [split][token][heads*dv].
template <typename T, int HPW>
__global__ void __launch_bounds__(kTalkWarps * 32)
talk_mix_kernel(const T* __restrict__ q, T* __restrict__ out, float* __restrict__ partial, const T* __restrict__ k_pool,
                const T* __restrict__ v_pool, const float* __restrict__ mix, const int* __restrict__ token_seq,
                const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
                int page_size, int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim, float scale,
                float out_scale, int split_keys, int num_splits, const float* __restrict__ stats) {
  extern __shared__ __align__(16) float shared[];
  TalkShared sh(shared, num_heads, head_dim);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < num_heads * num_heads; i += blockDim.x) sh.mix[i] = mix[i];
  pdl_wait();
  const int t = blockIdx.x, split = blockIdx.y;
  const int group = num_heads / num_kv_heads;
  const int position = positions[t];
  const int begin = split * split_keys, last = min(begin + split_keys - 1, position);
  if (begin > position) return;
  const int* table = block_table + static_cast<size_t>(token_seq[t]) * table_width;
  const T* q_row = q + static_cast<size_t>(t) * num_heads * head_dim;
  for (int i = threadIdx.x; i < num_heads * head_dim; i += blockDim.x) sh.q[i] = to_float<T>(q_row[i]);
  const int live_splits = position / split_keys + 1;
  for (int g = threadIdx.x; g < num_heads; g += blockDim.x) {
    const float* cell = stats + (static_cast<size_t>(t) * num_splits * num_heads + g) * 2;
    float whole_max = -INFINITY;
    for (int s = 0; s < live_splits; ++s) whole_max = fmaxf(whole_max, cell[static_cast<size_t>(s) * num_heads * 2]);
    float whole_sum = 0.0f;
    for (int s = 0; s < live_splits; ++s)
      whole_sum += cell[static_cast<size_t>(s) * num_heads * 2 + 1] * expf(cell[static_cast<size_t>(s) * num_heads * 2] - whole_max);
    sh.max[g] = whole_max;
    sh.inv[g] = 1.0f / whole_sum;
  }
  __syncthreads();
  const size_t k_stride = static_cast<size_t>(num_kv_heads) * head_dim;
  const size_t v_stride = static_cast<size_t>(num_kv_heads) * value_dim;
  float acc[HPW][kTalkMaxDim / 32];
#pragma unroll
  for (int s = 0; s < HPW; ++s)
#pragma unroll
    for (int i = 0; i < kTalkMaxDim / 32; ++i) acc[s][i] = 0.0f;
  for (int base = begin; base <= last; base += 32) {
    const int j = base + lane;
    const bool valid = j <= last;
    size_t at = 0;
    if (valid) at = static_cast<size_t>(table[j / page_size]) * page_size + j % page_size;
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
      const int g = warp + s * kTalkWarps;
      if (g >= num_heads) break;
      float p = 0.0f;
      if (valid) {
        const T* k_row = k_pool + at * k_stride + static_cast<size_t>(g / group) * head_dim;
        p = expf(talk_dot<T>(sh.q + g * head_dim, k_row, head_dim) * scale - sh.max[g]) * sh.inv[g];
      }
      sh.p[g * 32 + lane] = p;
    }
    __syncthreads();
    const int count = min(32, last - base + 1);
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
      const int h = warp + s * kTalkWarps;
      if (h >= num_heads) break;
      float weight = 0.0f;
      for (int g = 0; g < num_heads; ++g) weight = fmaf(sh.mix[h * num_heads + g], sh.p[g * 32 + lane], weight);
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
    const size_t at = (static_cast<size_t>(t) * num_heads + h) * value_dim;
#pragma unroll
    for (int i = 0; i < kTalkMaxDim / 32; ++i) {
      const int e = lane + 32 * i;
      if (e >= value_dim) continue;
      if (num_splits == 1) out[at + e] = from_float<T>(acc[s][i] * out_scale);
      else partial[static_cast<size_t>(split) * num_tokens * num_heads * value_dim + at + e] = acc[s][i];
    }
  }
}

// The splits' partial outputs added in order (only those that hold keys were written).
template <typename T>
__global__ void __launch_bounds__(256)
talk_sum_kernel(const float* __restrict__ partial, T* __restrict__ out, const int* __restrict__ positions, int num_tokens,
                int width, int split_keys, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int live_splits = positions[t] / split_keys + 1;
  for (int e = threadIdx.x; e < width; e += blockDim.x) {
    float sum = 0.0f;
    for (int s = 0; s < live_splits; ++s) sum += partial[(static_cast<size_t>(s) * num_tokens + t) * width + e];
    out[static_cast<size_t>(t) * width + e] = from_float<T>(sum * out_scale);
  }
}

template <typename T, int HPW>
static int launch_talk_sized(dim3 grid, size_t shared_bytes, cudaStream_t s, const void* q, void* out, const void* k_pool,
                             const void* v_pool, const float* mix, const int* token_seq, const int* positions,
                             const int* block_table, int table_width, int page_size, int num_heads, int num_kv_heads,
                             int head_dim, int value_dim, float scale, float out_scale, int split_keys, float* stats,
                             float* partial) {
  if (shared_bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(talk_stats_kernel<T, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(shared_bytes));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(talk_mix_kernel<T, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(shared_bytes));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int num_tokens = grid.x, num_splits = grid.y;
  int status = vipera_launch(talk_stats_kernel<T, HPW>, grid, kTalkWarps * 32, shared_bytes, s, static_cast<const T*>(q),
                             static_cast<const T*>(k_pool), token_seq, positions, block_table, table_width, page_size,
                             num_heads, num_kv_heads, head_dim, scale, split_keys, num_splits, stats);
  if (status) return status;
  status = vipera_launch(talk_mix_kernel<T, HPW>, grid, kTalkWarps * 32, shared_bytes, s, static_cast<const T*>(q),
                         static_cast<T*>(out), partial, static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), mix,
                         token_seq, positions, block_table, table_width, page_size, num_tokens, num_heads, num_kv_heads,
                         head_dim, value_dim, scale, out_scale, split_keys, num_splits, static_cast<const float*>(stats));
  if (status || num_splits == 1) return status;
  return vipera_launch(talk_sum_kernel<T>, dim3(num_tokens), 256, 0, s, static_cast<const float*>(partial),
                       static_cast<T*>(out), positions, num_tokens, num_heads * value_dim, split_keys, out_scale);
}

template <typename T>
static int launch_talk(int hpw, dim3 grid, size_t shared_bytes, cudaStream_t s, const void* q, void* out, const void* k_pool,
                       const void* v_pool, const float* mix, const int* token_seq, const int* positions,
                       const int* block_table, int table_width, int page_size, int num_heads, int num_kv_heads,
                       int head_dim, int value_dim, float scale, float out_scale, int split_keys, float* stats,
                       float* partial) {
#define TALK_CASE(N)                                                                                                  \
  return launch_talk_sized<T, N>(grid, shared_bytes, s, q, out, k_pool, v_pool, mix, token_seq, positions, block_table, \
                                 table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim, scale, out_scale, \
                                 split_keys, stats, partial);
  if (hpw <= 1) TALK_CASE(1)
  if (hpw <= 2) TALK_CASE(2)
  if (hpw <= 4) TALK_CASE(4)
  TALK_CASE(8)
#undef TALK_CASE
}

// q [tokens, heads, d], out [tokens, heads, value_dim], mix [heads, heads] 32-bit (row h holds the
// weights of head h's mix); pools and tables as in the general attention kernel.
// The mix applied to the 32-bit attention outputs of every (query head, KV head) pair: with a [tokens, heads *
// kv_heads, dv] = softmax(q_g k^T) v_c at row g * kv_heads + c, out[t, h] = out_scale * sum_g mix[h, g]
// a[t, g * kv_heads + kv(h)] (the same sum as mixing the weights, the values being shared).  32-bit sums.
template <typename T>
__global__ void __launch_bounds__(256)
talk_combine_kernel(const float* __restrict__ pairs, const float* __restrict__ mix, T* __restrict__ out, int num_heads,
                    int num_kv_heads, int value_dim, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int group = num_heads / num_kv_heads;
  const float* row = pairs + static_cast<size_t>(t) * num_heads * num_kv_heads * value_dim;
  for (int item = threadIdx.x; item < num_heads * value_dim; item += blockDim.x) {
    const int h = item / value_dim, e = item % value_dim;
    const int kv = h / group;
    float sum = 0.0f;
    for (int g = 0; g < num_heads; ++g)
      sum = fmaf(mix[h * num_heads + g], row[(static_cast<size_t>(g) * num_kv_heads + kv) * value_dim + e], sum);
    out[static_cast<size_t>(t) * num_heads * value_dim + item] = from_float<T>(sum * out_scale);
  }
}

VIPERA_API int vipera_talk_combine(const float* pairs, const float* mix, void* out, int dtype, int num_tokens,
                                   int num_heads, int num_kv_heads, int value_dim, float out_scale, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || value_dim <= 0) return VIPERA_BAD_SHAPE;
  if (!pairs || !mix || !out) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == VIPERA_BF16)
    return vipera_launch(talk_combine_kernel<__nv_bfloat16>, dim3(num_tokens), 256, 0, s,
                         pairs, mix, static_cast<__nv_bfloat16*>(out), num_heads, num_kv_heads, value_dim, out_scale);
  if (dtype == VIPERA_F32)
    return vipera_launch(talk_combine_kernel<float>, dim3(num_tokens), 256, 0, s, pairs, mix, static_cast<float*>(out),
                         num_heads, num_kv_heads, value_dim, out_scale);
  return VIPERA_BAD_DTYPE;
}

// The keys are cut into `num_splits` splits of `split_keys` keys (a multiple of 32) so that steps of
// few tokens still fill the GPU: `stats` holds 2 * tokens * splits * heads floats, `partial`
// splits * tokens * heads * value_dim floats (not used with one split).
VIPERA_API int vipera_attention_talk(const void* q, void* out, int dtype, const void* k_pool, const void* v_pool,
                                     const float* mix, const int* token_seq, const int* positions,
                                     const int* block_table, int table_width, int page_size, int num_tokens,
                                     int num_heads, int num_kv_heads, int head_dim, int value_dim, float scale,
                                     float out_scale, int split_keys, int num_splits, float* stats, float* partial,
                                     void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (head_dim <= 0 || head_dim > kTalkMaxDim || value_dim <= 0 || value_dim > kTalkMaxDim) return VIPERA_BAD_SHAPE;
  if (num_heads <= 0 || num_heads > kTalkMaxHeads || num_kv_heads <= 0 || num_heads % num_kv_heads) return VIPERA_BAD_SHAPE;
  if (page_size <= 0 || table_width <= 0 || !mix || !stats) return VIPERA_BAD_ARGUMENT;
  if (num_splits < 1 || num_splits > 65535 || split_keys < 32 || split_keys % 32 || (num_splits > 1 && !partial))
    return VIPERA_BAD_ARGUMENT;
  const size_t shared_bytes = sizeof(float) * (static_cast<size_t>(num_heads) * head_dim + num_heads * num_heads +
                                               num_heads * 32 + 2 * num_heads);
  if (shared_bytes > 200 * 1024) return VIPERA_BAD_SHAPE;
  const int hpw = (num_heads + kTalkWarps - 1) / kTalkWarps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tokens, num_splits);
  if (dtype == VIPERA_F32)
    return launch_talk<float>(hpw, grid, shared_bytes, s, q, out, k_pool, v_pool, mix, token_seq, positions, block_table,
                              table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim, scale, out_scale,
                              split_keys, stats, partial);
  if (dtype == VIPERA_BF16)
    return launch_talk<__nv_bfloat16>(hpw, grid, shared_bytes, s, q, out, k_pool, v_pool, mix, token_seq, positions,
                                      block_table, table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim,
                                      scale, out_scale, split_keys, stats, partial);
  return VIPERA_BAD_DTYPE;
}
