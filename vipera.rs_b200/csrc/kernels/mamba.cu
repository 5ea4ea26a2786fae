// Mamba's selective scan over a step's flattened tokens, with each request's state kept between
// steps.  Per channel c and state index n, for every token of a request in order:
//
//   dt      = softplus(dt_pre[t, c])                       (dt_pre: the step-size product, bias included)
//   S[c, n] = exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n]
//   y[t, c] = sum_n S[c, n] * C[t, n] + D[c] * x[t, c]
//   out     = y * silu(z[t, c])
//
// A = -exp(A_log) is formed once when the model is built.  S lives in 32-bit floats,
// [slots, channels, states], starts at zero for a new request and is carried from portion to
// portion.  Everything here is 32-bit arithmetic; only `out` takes the run's type.
//
// A channel is shared by LANES adjacent lanes of a warp (a power of two), each holding NPL states
// in registers; the sum over n is a shuffle reduction.  A block covers kScanThreads / LANES
// channels of one entry and walks the entry's tokens in order.  The same kernel serves portions
// and single tokens.
//
// Long steps are cut into chunks of kScanChunk tokens that run side by side, in three launches:
// every chunk from a zero state (its end state E and the sum of its step sizes, which gives the
// chunk's whole decay exp(A * sum dt)); per entry the states at the chunks' starts, one after
// another, S <- exp(A * sum dt) * S + E, which also leaves the request's new state; every chunk
// again from its start state, now with outputs.  The recurrence is linear in S, so this only
// re-associates 32-bit sums.  Chunks are counted from where an entry's tokens start in the step.
#include "common.cuh"

#include <algorithm>

constexpr int kScanThreads = 128;

struct ScanParams {
  const float* x;        // [tokens, channels]   conv + silu output
  const float* dt_pre;   // [tokens, channels]
  const float* bc;       // [tokens, 2 * states]  B then C
  const float* z;        // [tokens, z_stride]    the gate's pre-activation at column z_offset
  long long z_stride;
  int z_offset;
  const float* a;        // [channels, states]    negative
  const float* d;        // [channels]
  float* state;          // [slots, channels * states]
  const int* entry_starts;
  const int* state_slots;
  const int* fresh;
  void* out;             // [tokens, channels]
  int channels, states, num_entries, lanes;
  // the chunked form: mode 0 walks whole entries; 1 runs chunks from zero; 3 runs them from their start states
  int mode, num_jobs;
  float* chunk_state;    // [jobs, channels * states]  end states (mode 1), then start states (mode 3)
  float* chunk_dt;       // [jobs, channels]           sums of the chunks' step sizes
};

constexpr int kScanChunk = 64;

// Which (entry, first token, end) is job `job`: the entries' chunks are numbered one entry after another.
__device__ __forceinline__ bool scan_job(const int* __restrict__ entry_starts, int num_entries, int job, int* entry,
                                         int* first, int* last) {
  int before = 0;
  for (int e = 0; e < num_entries; ++e) {
    const int begin = entry_starts[e], count = entry_starts[e + 1] - begin;
    const int chunks = (count + kScanChunk - 1) / kScanChunk;
    if (job < before + chunks) {
      *entry = e;
      *first = begin + (job - before) * kScanChunk;
      *last = min(*first + kScanChunk, begin + count);
      return true;
    }
    before += chunks;
  }
  return false;
}

// Tokens are staged in shared memory `tile` at a time by the whole block: the step sizes (softplus
// applied once per token and channel), x and the gate of the block's channels, and the B and C
// rows; the walk over the tokens then reads shared memory only.
// exp for the decays and the gate: the library's in a 32-bit run; in a bfloat16 run the hardware's
// approximation (a few units in the last place of a 32-bit float, far below that run's rounding).
template <typename TO>
__device__ __forceinline__ float scan_exp(float v) { return expf(v); }
template <>
__device__ __forceinline__ float scan_exp<__nv_bfloat16>(float v) { return __expf(v); }

// ENDS: the pass that only finds the chunks' end states (mode 1): no C rows, no gate, no outputs.
template <typename TO, int NPL, bool ENDS>
__global__ void __launch_bounds__(kScanThreads) mamba_scan_kernel(const ScanParams p, int tile) {
  extern __shared__ __align__(16) float staged[];
  pdl_launch_dependents();
  const int lanes = p.lanes;
  const int per_block = kScanThreads / lanes;               // channels of a block
  const int sub = threadIdx.x % lanes;                      // which share of the states
  const int local = threadIdx.x / lanes;
  const int c0 = blockIdx.x * per_block;
  const int c = c0 + local;
  const bool live = c < p.channels;
  int entry = blockIdx.y;
  float* dt_s = staged;                                     // [tile][per_block]
  float* x_s = dt_s + tile * per_block;
  float* z_s = x_s + tile * per_block;
  float* bc_s = z_s + tile * per_block;                     // [tile][2 * states]
  float a[NPL], s[NPL];
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int n = sub * NPL + j;
    a[j] = (live && n < p.states) ? p.a[static_cast<size_t>(c) * p.states + n] : 0.0f;
    s[j] = 0.0f;
  }
  const float skip = live ? p.d[c] : 0.0f;
  pdl_wait();
  int first, last;
  float* state;
  bool resume;
  if (p.mode == 0) {
    first = p.entry_starts[entry];
    last = p.entry_starts[entry + 1];
    if (last <= first) return;
    state = p.state + static_cast<size_t>(p.state_slots[entry]) * p.channels * p.states;
    resume = !p.fresh[entry];
  } else {
    if (!scan_job(p.entry_starts, p.num_entries, blockIdx.y, &entry, &first, &last)) return;
    state = p.chunk_state + static_cast<size_t>(blockIdx.y) * p.channels * p.states;
    resume = p.mode == 3;
  }
  if (live && resume) {
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      const int n = sub * NPL + j;
      if (n < p.states) s[j] = state[static_cast<size_t>(c) * p.states + n];
    }
  }
  TO* out = static_cast<TO*>(p.out);
  float dt_sum = 0.0f;
  const int width = 2 * p.states;
  const bool vector_rows = (p.states & 3) == 0 && ((3 * tile * per_block) & 3) == 0;
  for (int t0 = first; t0 < last; t0 += tile) {
    const int count = min(tile, last - t0);
    __syncthreads();
    for (int index = threadIdx.x; index < count * per_block; index += kScanThreads) {
      const int tt = index / per_block, cl = index % per_block;
      const bool valid = c0 + cl < p.channels;
      const size_t at = static_cast<size_t>(t0 + tt) * p.channels + c0 + cl;
      const float pre = valid ? p.dt_pre[at] : 0.0f;
      dt_s[index] = pre > 20.0f ? pre : log1pf(expf(pre));
      x_s[index] = valid ? p.x[at] : 0.0f;
      if (!ENDS) z_s[index] = valid ? p.z[static_cast<size_t>(t0 + tt) * p.z_stride + p.z_offset + c0 + cl] : 0.0f;
    }
    for (int index = threadIdx.x; index < count * width; index += kScanThreads)
      bc_s[index] = p.bc[static_cast<size_t>(t0) * width + index];
    __syncthreads();
    for (int tt = 0; tt < count; ++tt) {
      const float dt = dt_s[tt * per_block + local];
      const float x = x_s[tt * per_block + local];
      const float* b_row = bc_s + tt * width;
      const float* c_row = b_row + p.states;
      const float dtx = dt * x;
      dt_sum += dt;
      float y = 0.0f;
      if (NPL == 4 && vector_rows) {
        // four states a lane, rows of B and C that start on 16 bytes: one read each
        if (sub * 4 < p.states) {
          const float4 b4 = *reinterpret_cast<const float4*>(b_row + sub * 4);
          s[0] = fmaf(scan_exp<TO>(dt * a[0]), s[0], dtx * b4.x);
          s[1 % NPL] = fmaf(scan_exp<TO>(dt * a[1 % NPL]), s[1 % NPL], dtx * b4.y);
          s[2 % NPL] = fmaf(scan_exp<TO>(dt * a[2 % NPL]), s[2 % NPL], dtx * b4.z);
          s[3 % NPL] = fmaf(scan_exp<TO>(dt * a[3 % NPL]), s[3 % NPL], dtx * b4.w);
          if (!ENDS) {
            const float4 c4 = *reinterpret_cast<const float4*>(c_row + sub * 4);
            y = fmaf(s[0], c4.x, y);
            y = fmaf(s[1 % NPL], c4.y, y);
            y = fmaf(s[2 % NPL], c4.z, y);
            y = fmaf(s[3 % NPL], c4.w, y);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < NPL; ++j) {
          const int n = sub * NPL + j;
          if (n < p.states) {
            s[j] = fmaf(scan_exp<TO>(dt * a[j]), s[j], dtx * b_row[n]);
            if (!ENDS) y = fmaf(s[j], c_row[n], y);
          }
        }
      }
      if (!ENDS) {
        for (int offset = lanes >> 1; offset > 0; offset >>= 1) y += __shfl_xor_sync(0xffffffffu, y, offset);
        if (live && sub == 0) {
          const float gate = z_s[tt * per_block + local];
          y = fmaf(skip, x, y);
          out[static_cast<size_t>(t0 + tt) * p.channels + c] = from_float<TO>(y * (gate / (1.0f + scan_exp<TO>(-gate))));
        }
      }
    }
  }
  if (live && p.mode != 3) {
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      const int n = sub * NPL + j;
      if (n < p.states) state[static_cast<size_t>(c) * p.states + n] = s[j];
    }
    if (p.mode == 1 && sub == 0) p.chunk_dt[static_cast<size_t>(blockIdx.y) * p.channels + c] = dt_sum;
  }
}

// Between the two chunk passes: per entry and state element, the states at the chunks' starts one
// after another (they take the end states' places), and the request's new state.
__global__ void __launch_bounds__(kScanThreads) mamba_chunk_starts_kernel(const ScanParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t width = static_cast<size_t>(p.channels) * p.states;
  const size_t item = static_cast<size_t>(blockIdx.x) * kScanThreads + threadIdx.x;
  const int entry = blockIdx.y;
  if (item >= width) return;
  const int begin = p.entry_starts[entry], count = p.entry_starts[entry + 1] - begin;
  if (count <= 0) return;
  int job = 0;
  for (int e = 0; e < entry; ++e) job += (p.entry_starts[e + 1] - p.entry_starts[e] + kScanChunk - 1) / kScanChunk;
  const int chunks = (count + kScanChunk - 1) / kScanChunk;
  const int c = static_cast<int>(item / p.states);
  const float a = p.a[item];
  float* state = p.state + static_cast<size_t>(p.state_slots[entry]) * width + item;
  float s = p.fresh[entry] ? 0.0f : *state;
  for (int k = 0; k < chunks; ++k, ++job) {
    float* cell = p.chunk_state + static_cast<size_t>(job) * width + item;
    const float end_state = *cell;
    *cell = s;
    s = fmaf(expf(a * p.chunk_dt[static_cast<size_t>(job) * p.channels + c]), s, end_state);
  }
  *state = s;
}

// How the states of a channel are dealt to lanes: (lanes, states per lane), at most
// `most_per_lane` states a lane.  (Sixteen a lane in the chunked form, whose chunks fill the GPU
// anyway, was measured: 15 % slower at 3,072 channels, 3 % faster at 8,192; four it stays.)
static void scan_shape(int states, int most_per_lane, int* lanes, int* per_lane) {
  int l = 1;
  while (l < 32 && (states + l - 1) / l > most_per_lane) l *= 2;
  *lanes = l;
  const int need = (states + l - 1) / l;
  *per_lane = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : 16;
}

VIPERA_API int vipera_mamba_scan(const ScanParams* params, int out_dtype, void* stream) {
  ScanParams p = *params;
  if (p.num_entries <= 0) return VIPERA_OK;
  if (p.channels <= 0 || p.states <= 0 || p.states > 512) return VIPERA_BAD_SHAPE;
  if (!p.x || !p.dt_pre || !p.bc || !p.z || !p.a || !p.d || !p.state || !p.entry_starts || !p.state_slots ||
      !p.fresh || !p.out)
    return VIPERA_BAD_ARGUMENT;
  int per_lane = 1;
  const bool chunked = p.num_jobs > 0 && p.chunk_state && p.chunk_dt;
  scan_shape(p.states, 4, &p.lanes, &per_lane);
  const int channels_per_block = kScanThreads / p.lanes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype != VIPERA_BF16 && out_dtype != VIPERA_F32) return VIPERA_BAD_DTYPE;
  // tokens staged at a time: what fits 16 KB beside the block's channels (so that an SM holds a
  // dozen blocks), at most half a chunk
  const size_t per_token = (3 * static_cast<size_t>(channels_per_block) + 2 * p.states) * sizeof(float);
  const int tile = static_cast<int>(std::max<size_t>(1, std::min<size_t>(kScanChunk / 2, (16 * 1024) / per_token)));
  const size_t shared_bytes = tile * per_token;
  auto pass = [&](int mode) -> int {
    p.mode = mode;
    dim3 grid((p.channels + channels_per_block - 1) / channels_per_block, mode == 0 ? p.num_entries : p.num_jobs);
#define SCAN_CASE(N)                                                                                     \
  if (per_lane == N) {                                                                                   \
    if (mode == 1) {                                                                                     \
      if (out_dtype == VIPERA_BF16)                                                                      \
        return vipera_launch(mamba_scan_kernel<__nv_bfloat16, N, true>, grid, kScanThreads, shared_bytes, s, p, tile); \
      return vipera_launch(mamba_scan_kernel<float, N, true>, grid, kScanThreads, shared_bytes, s, p, tile); \
    }                                                                                                    \
    if (out_dtype == VIPERA_BF16)                                                                        \
      return vipera_launch(mamba_scan_kernel<__nv_bfloat16, N, false>, grid, kScanThreads, shared_bytes, s, p, tile); \
    return vipera_launch(mamba_scan_kernel<float, N, false>, grid, kScanThreads, shared_bytes, s, p, tile); \
  }
    SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(16)
#undef SCAN_CASE
    return VIPERA_BAD_SHAPE;
  };
  if (!chunked) return pass(0);
  int status = pass(1);
  if (status) return status;
  const size_t width = static_cast<size_t>(p.channels) * p.states;
  status = vipera_launch(mamba_chunk_starts_kernel, dim3(static_cast<unsigned>((width + kScanThreads - 1) / kScanThreads), p.num_entries),
                         kScanThreads, 0, s, p);
  if (status) return status;
  return pass(3);
}

VIPERA_API int vipera_mamba_scan_chunk() { return kScanChunk; }

VIPERA_API int vipera_mamba_scan_params_size() { return static_cast<int>(sizeof(ScanParams)); }
