// A short causal convolution over time, one filter per channel, over a step's flattened tokens,
// with each request's last inputs kept between steps.
//
//   y[t, c] = act(sum_j w[c, j] * x[t - taps + 1 + j, c] + b[c]) (+ x[t, c])
//
// The last column of w is the current token's; inputs before a request's first token are zero.
// The state of a request is its last taps - 1 inputs, 32-bit, [taps - 1, channels], oldest first;
// a portion of a prompt continues from it.  Only the first taps - 1 tokens of an entry read the
// state and only the entry's end defines the new one, so one thread per (entry, channel) does
// both (reads the old rows into registers, computes those tokens, writes the new rows) and no
// other thread touches that state: the "head" jobs.  All other tokens read their inputs from the
// step's own rows: the "segment" jobs.  An entry without tokens leaves its state alone.
#include "common.cuh"

constexpr int kConvMaxTaps = 16;
constexpr int kConvThreads = 128;
constexpr int kConvSegment = 8;   // tokens of a segment job

enum ConvActivation { CONV_ACT_NONE = 0, CONV_ACT_SILU = 1 };

struct ConvParams {
  const float* x;          // [tokens, x_stride]; the first `channels` columns count
  long long x_stride;
  const float* weight;     // [channels, taps]
  const float* bias;       // [channels] or null
  float* state;            // [slots, state_stride] or null (taps == 1)
  long long state_stride;
  const int* entry_starts;
  const int* token_entry;
  const int* state_slots;
  const int* fresh;
  void* out;               // [tokens, channels] in the run's type, or null
  float* out_f32;          // [tokens, channels] or null
  float* clear;            // [tokens, channels] set to zero, or null
  int channels, taps, num_tokens, num_entries, add_input, activation, segments;
};

__device__ __forceinline__ float conv_finish(float sum, float current, const ConvParams& p, float bias) {
  sum += bias;
  if (p.activation == CONV_ACT_SILU) sum = sum / (1.0f + expf(-sum));
  if (p.add_input) sum += current;
  return sum;
}

template <typename TO>
__device__ __forceinline__ void conv_store(const ConvParams& p, int t, int c, float value) {
  const size_t at = static_cast<size_t>(t) * p.channels + c;
  if (p.out) static_cast<TO*>(p.out)[at] = from_float<TO>(value);
  if (p.out_f32) p.out_f32[at] = value;
  if (p.clear) p.clear[at] = 0.0f;
}

// MAXT: the most taps this instance takes (its register arrays and unrolled loops are that long).
template <typename TO, int MAXT>
__global__ void __launch_bounds__(kConvThreads) causal_conv_kernel(const ConvParams p) {
  pdl_launch_dependents();
  const int c = blockIdx.x * kConvThreads + threadIdx.x;
  const bool live = c < p.channels;
  const int taps = p.taps;
  float w[MAXT];
#pragma unroll
  for (int j = 0; j < MAXT; ++j) w[j] = (live && j < taps) ? p.weight[static_cast<size_t>(c) * taps + j] : 0.0f;
  const float bias = (live && p.bias) ? p.bias[c] : 0.0f;
  pdl_wait();
  if (!live) return;
  const int job = blockIdx.y;
  if (job < p.num_entries) {
    // head job: the entry's first taps - 1 tokens and its new state
    const int first = p.entry_starts[job], count = p.entry_starts[job + 1] - first;
    if (count <= 0) return;
    float old[MAXT];   // old[k], k < taps - 1: the input at in-entry index k - (taps - 1)
#pragma unroll
    for (int k = 0; k < MAXT; ++k) old[k] = 0.0f;
    float* state = nullptr;
    if (p.state && taps > 1) {
      state = p.state + static_cast<size_t>(p.state_slots[job]) * p.state_stride;
      if (!p.fresh[job]) {
#pragma unroll
        for (int k = 0; k < MAXT - 1; ++k)
          if (k < taps - 1) old[k] = state[static_cast<size_t>(k) * p.channels + c];
      }
    }
    const int heads = min(count, taps - 1);
    for (int i = 0; i < heads; ++i) {
      float sum = 0.0f, current = 0.0f;
#pragma unroll
      for (int j = 0; j < MAXT; ++j) {
        if (j < taps) {
          const int index = i - (taps - 1) + j;   // in-entry index of the input
          float value;
          if (index >= 0) value = p.x[static_cast<size_t>(first + index) * p.x_stride + c];
          else {
            value = 0.0f;
#pragma unroll
            for (int k = 0; k < MAXT - 1; ++k) if (k == taps - 1 + index) value = old[k];
          }
          sum = fmaf(w[j], value, sum);
          if (j == taps - 1) current = value;
        }
      }
      conv_store<TO>(p, first + i, c, conv_finish(sum, current, p, bias));
    }
    if (state) {
#pragma unroll
      for (int k = 0; k < MAXT - 1; ++k) {
        if (k < taps - 1) {
          const int index = count - (taps - 1) + k;
          float value;
          if (index >= 0) value = p.x[static_cast<size_t>(first + index) * p.x_stride + c];
          else {
            value = 0.0f;
#pragma unroll
            for (int m = 0; m < MAXT - 1; ++m) if (m == taps - 1 + index) value = old[m];
          }
          state[static_cast<size_t>(k) * p.channels + c] = value;
        }
      }
    }
    return;
  }
  // segment job: tokens far enough into their entry to read only the step's own rows
  const int begin = (job - p.num_entries) * kConvSegment;
  const int end = min(begin + kConvSegment, p.num_tokens);
  for (int t = begin; t < end; ++t) {
    const int entry = p.token_entry[t];
    const int index = t - p.entry_starts[entry];
    if (index < taps - 1) continue;
    float sum = 0.0f, current = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
      if (j < taps) {
        const float value = p.x[static_cast<size_t>(t - (taps - 1) + j) * p.x_stride + c];
        sum = fmaf(w[j], value, sum);
        if (j == taps - 1) current = value;
      }
    }
    conv_store<TO>(p, t, c, conv_finish(sum, current, p, bias));
  }
}

// single != 0 promises that every entry brings at most one token (no segment jobs are needed
// when taps > 1).
VIPERA_API int vipera_causal_conv(const ConvParams* params, int out_dtype, int single, void* stream) {
  ConvParams p = *params;
  if (p.num_tokens <= 0) return VIPERA_OK;
  if (p.channels <= 0 || p.taps < 1 || p.taps > kConvMaxTaps) return VIPERA_BAD_SHAPE;
  if (!p.x || !p.weight || !p.entry_starts || !p.token_entry || p.num_entries <= 0) return VIPERA_BAD_ARGUMENT;
  if (p.taps > 1 && p.state && (!p.state_slots || !p.fresh)) return VIPERA_BAD_ARGUMENT;
  p.segments = (single && p.taps > 1) ? 0 : (p.num_tokens + kConvSegment - 1) / kConvSegment;
  dim3 grid((p.channels + kConvThreads - 1) / kConvThreads, p.num_entries + p.segments);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype != VIPERA_BF16 && out_dtype != VIPERA_F32) return VIPERA_BAD_DTYPE;
#define CONV_CASE(N)                                                                                          \
  if (p.taps <= N) {                                                                                          \
    if (out_dtype == VIPERA_BF16) return vipera_launch(causal_conv_kernel<__nv_bfloat16, N>, grid, kConvThreads, 0, s, p); \
    return vipera_launch(causal_conv_kernel<float, N>, grid, kConvThreads, 0, s, p);                          \
  }
  CONV_CASE(4) CONV_CASE(8) CONV_CASE(kConvMaxTaps)
#undef CONV_CASE
  return VIPERA_BAD_SHAPE;
}

VIPERA_API int vipera_causal_conv_params_size() { return static_cast<int>(sizeof(ConvParams)); }
