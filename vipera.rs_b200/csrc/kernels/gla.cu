// Gated linear attention over a step's flattened tokens, with each request's state kept between
// steps.  Per head, with S a matrix [d, dv] (rows belong to key channels):
//
//   alpha_t = sigmoid(z_t)^(1 / tau)         one decay per key channel, z the decay product
//   S_t     = diag(alpha_t) S_(t-1) + k_t v_t^T
//   o_t     = S_t^T (q_t * q_scale)
//
// then each head's o is divided by its root mean square over dv (sqrt(mean + eps)), multiplied
// by a weight per value (shared by the heads), by silu of the output gate g and by `out_scale`.
// S lives in 32-bit floats, [slots, heads, d, dv], starts at zero for a new request and is
// carried from portion to portion.  Decays (through log sigmoid), state, products with the state
// and the norm are 32-bit.
//
// gla_decay_kernel forms the decays and their logarithms once per token and key channel.
// gla_scan_kernel: a block owns (ROWS rows of the state: a "share", up to eight tiles of 32 value
// columns, head, entry or chunk) and walks the tokens in order (see there).  Each share writes its
// part of o to a scratch [row shares][tokens][heads*dv]; gla_finish_kernel adds the shares in a
// fixed order and applies norm, gate and scale (a warp per (token, head)).
//
// Long steps are cut into chunks of kGlaChunk tokens that run side by side, in three launches:
// every chunk from a zero state (its end state E and, per key channel, the sum of its log decays,
// which gives the chunk's whole decay); per entry the states at the chunks' starts one after
// another, S <- exp(sum log alpha) S + E, which also leaves the request's new state; every chunk
// again from its start state, now with outputs.  The recurrence is linear in S, so this only
// re-associates 32-bit sums.  Chunks are counted from where an entry's tokens start in the step.
#include "common.cuh"

#include <algorithm>

constexpr int kGlaMaxShares = 16;

struct GlaParams {
  const float* proj;      // [tokens, proj_width]: q, k, v, g at their offsets
  long long proj_width;
  int q_off, k_off, v_off, g_off;
  float* z;               // [tokens, heads * dim]  decay pre-activations (bias included); the decays take their place
  float* log_alpha;       // [tokens, heads * dim]  receives the decays' logarithms
  float* state;           // [slots, heads * dim * vdim]
  const int* entry_starts;
  const int* state_slots;
  const int* fresh;
  float* partial;         // [shares][tokens][heads * vdim]
  const float* norm_weight;  // [vdim]
  void* out;              // [tokens, heads * vdim]
  int heads, dim, vdim, num_entries, num_tokens, shares;
  float q_scale, inv_tau, eps, out_scale;
  // the chunked form: mode 0 walks whole entries; 1 runs chunks from zero; 3 runs them from their start states
  int mode, num_jobs;
  float* chunk_state;     // [jobs, heads * dim * vdim]  end states (mode 1), then start states (mode 3)
  float* chunk_decay;     // [jobs, heads * dim]         sums of the chunks' log decays
};

constexpr int kGlaChunk = 64;

__device__ __forceinline__ bool gla_job(const int* __restrict__ entry_starts, int num_entries, int job, int* entry,
                                        int* first, int* last) {
  int before = 0;
  for (int e = 0; e < num_entries; ++e) {
    const int begin = entry_starts[e], count = entry_starts[e + 1] - begin;
    const int chunks = (count + kGlaChunk - 1) / kGlaChunk;
    if (job < before + chunks) {
      *entry = e;
      *first = begin + (job - before) * kGlaChunk;
      *last = min(*first + kGlaChunk, begin + count);
      return true;
    }
    before += chunks;
  }
  return false;
}

// alpha = sigmoid(z)^(1 / tau) through log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)), once per token
// and key channel: alpha takes z's place, its logarithm goes beside it.
__global__ void __launch_bounds__(256) gla_decay_kernel(const GlaParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t count = static_cast<size_t>(p.num_tokens) * p.heads * p.dim;
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < count; i += static_cast<size_t>(gridDim.x) * 256) {
    const float zz = p.z[i];
    const float log_alpha = (fminf(zz, 0.0f) - log1pf(expf(-fabsf(zz)))) * p.inv_tau;
    p.log_alpha[i] = log_alpha;
    p.z[i] = expf(log_alpha);
  }
}

constexpr int kGlaTile = 64;      // tokens whose decays, keys and queries a block stages at a time
constexpr int kGlaWarps = 8;      // value tiles (of 32 columns) a block covers

// A block owns ROWS rows of a head's state (a "share") for up to kGlaWarps tiles of 32 value
// columns: a warp a tile, a lane a column, the rows in registers.  The rows' decays, keys and
// scaled queries of kGlaTile tokens at a time are staged in shared memory by the whole block (they
// are the same for every column); a token then costs a warp one coalesced load of v, broadcast
// reads of the staged rows, and 2 * ROWS multiply-adds.
// ENDS: the pass that only finds the chunks' end states (mode 1): no queries, no outputs.
template <int ROWS, bool ENDS>
__global__ void __launch_bounds__(kGlaWarps * 32) gla_scan_kernel(const GlaParams p) {
  __shared__ __align__(16) float staged[ENDS ? 2 : 3][kGlaTile][ROWS];   // decays, keys, queries
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int share = blockIdx.x % p.shares, tiles0 = (blockIdx.x / p.shares) * kGlaWarps;
  const int column = (tiles0 + warp) * 32 + lane;
  const int head = blockIdx.y;
  int entry = blockIdx.z;
  const bool live = column < p.vdim;
  const int row0 = share * ROWS;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) s[r] = 0.0f;
  pdl_wait();
  int first, last;
  float* state;
  bool resume;
  if (p.mode == 0) {
    first = p.entry_starts[entry];
    last = p.entry_starts[entry + 1];
    if (last <= first) return;
    state = p.state + (static_cast<size_t>(p.state_slots[entry]) * p.heads + head) * p.dim * p.vdim;
    resume = !p.fresh[entry];
  } else {
    if (!gla_job(p.entry_starts, p.num_entries, blockIdx.z, &entry, &first, &last)) return;
    state = p.chunk_state + (static_cast<size_t>(blockIdx.z) * p.heads + head) * p.dim * p.vdim;
    resume = p.mode == 3;
  }
  if (live && resume) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < p.dim) s[r] = state[static_cast<size_t>(row0 + r) * p.vdim + column];
  }
  const size_t out_width = static_cast<size_t>(p.heads) * p.vdim;
  float* partial = p.partial + static_cast<size_t>(share) * p.num_tokens * out_width + head * p.vdim;
  const float* v_column = p.proj + p.v_off + head * p.vdim + (live ? column : 0);
  for (int t0 = first; t0 < last; t0 += kGlaTile) {
    const int count = min(kGlaTile, last - t0);
    __syncthreads();
    for (int index = threadIdx.x; index < count * ROWS; index += blockDim.x) {
      const int tt = index / ROWS, r = index % ROWS;
      const bool valid = row0 + r < p.dim;
      const float* row = p.proj + static_cast<size_t>(t0 + tt) * p.proj_width + head * p.dim + row0 + r;
      staged[0][tt][r] = valid ? p.z[(static_cast<size_t>(t0 + tt) * p.heads + head) * p.dim + row0 + r] : 0.0f;
      staged[1][tt][r] = valid ? row[p.k_off] : 0.0f;
      if (!ENDS) staged[2][tt][r] = valid ? row[p.q_off] * p.q_scale : 0.0f;
    }
    __syncthreads();
    float v_next = v_column[static_cast<size_t>(t0) * p.proj_width];
    for (int tt = 0; tt < count; ++tt) {
      const float v = live ? v_next : 0.0f;
      if (tt + 1 < count) v_next = v_column[static_cast<size_t>(t0 + tt + 1) * p.proj_width];
      float o = 0.0f;
#pragma unroll
      for (int r = 0; r < ROWS; r += 4) {
        const float4 alpha = *reinterpret_cast<const float4*>(&staged[0][tt][r]);
        const float4 k = *reinterpret_cast<const float4*>(&staged[1][tt][r]);
        s[r] = fmaf(alpha.x, s[r], k.x * v);
        s[r + 1] = fmaf(alpha.y, s[r + 1], k.y * v);
        s[r + 2] = fmaf(alpha.z, s[r + 2], k.z * v);
        s[r + 3] = fmaf(alpha.w, s[r + 3], k.w * v);
        if (!ENDS) {
          const float4 q = *reinterpret_cast<const float4*>(&staged[ENDS ? 0 : 2][tt][r]);
          o = fmaf(s[r], q.x, o);
          o = fmaf(s[r + 1], q.y, o);
          o = fmaf(s[r + 2], q.z, o);
          o = fmaf(s[r + 3], q.w, o);
        }
      }
      if (!ENDS && live) partial[static_cast<size_t>(t0 + tt) * out_width + column] = o;
    }
  }
  if (live && p.mode != 3) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < p.dim) state[static_cast<size_t>(row0 + r) * p.vdim + column] = s[r];
  }
  if (p.mode == 1 && blockIdx.x < p.shares && threadIdx.x < ROWS && row0 + threadIdx.x < p.dim) {
    // the chunk's whole decay per key channel: the sum of its log decays, in token order
    float sum = 0.0f;
    for (int t = first; t < last; ++t)
      sum += p.log_alpha[(static_cast<size_t>(t) * p.heads + head) * p.dim + row0 + threadIdx.x];
    p.chunk_decay[(static_cast<size_t>(blockIdx.z) * p.heads + head) * p.dim + row0 + threadIdx.x] = sum;
  }
}

// Between the two chunk passes: per entry and state element, the states at the chunks' starts one
// after another (they take the end states' places), and the request's new state.
__global__ void __launch_bounds__(256) gla_chunk_starts_kernel(const GlaParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t width = static_cast<size_t>(p.heads) * p.dim * p.vdim;
  const size_t item = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const int entry = blockIdx.y;
  if (item >= width) return;
  const int begin = p.entry_starts[entry], count = p.entry_starts[entry + 1] - begin;
  if (count <= 0) return;
  int job = 0;
  for (int e = 0; e < entry; ++e) job += (p.entry_starts[e + 1] - p.entry_starts[e] + kGlaChunk - 1) / kGlaChunk;
  const int chunks = (count + kGlaChunk - 1) / kGlaChunk;
  const size_t row = item / p.vdim;   // head * dim + key channel
  float* state = p.state + static_cast<size_t>(p.state_slots[entry]) * width + item;
  float s = p.fresh[entry] ? 0.0f : *state;
  for (int k = 0; k < chunks; ++k, ++job) {
    float* cell = p.chunk_state + static_cast<size_t>(job) * width + item;
    const float end_state = *cell;
    *cell = s;
    s = fmaf(expf(p.chunk_decay[static_cast<size_t>(job) * p.heads * p.dim + row]), s, end_state);
  }
  *state = s;
}

template <typename TO>
__global__ void __launch_bounds__(128) gla_finish_kernel(const GlaParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= p.num_tokens * p.heads) return;
  const int t = item / p.heads, head = item % p.heads;
  const size_t out_width = static_cast<size_t>(p.heads) * p.vdim;
  const size_t base = static_cast<size_t>(t) * out_width + head * p.vdim;
  float squares = 0.0f;
  for (int e = lane; e < p.vdim; e += 32) {
    float o = 0.0f;
    for (int share = 0; share < p.shares; ++share) o += p.partial[static_cast<size_t>(share) * p.num_tokens * out_width + base + e];
    p.partial[base + e] = o;   // share 0 now holds the sum (this lane alone reads and writes it)
    squares = fmaf(o, o, squares);
  }
  const float inverse = 1.0f / sqrtf(warp_sum(squares) / static_cast<float>(p.vdim) + p.eps);
  const float* gate = p.proj + static_cast<size_t>(t) * p.proj_width + p.g_off + head * p.vdim;
  TO* out = static_cast<TO*>(p.out) + base;
  for (int e = lane; e < p.vdim; e += 32) {
    const float g = gate[e];
    out[e] = from_float<TO>(p.partial[base + e] * inverse * p.norm_weight[e] * (g / (1.0f + expf(-g))) * p.out_scale);
  }
}

// Rows of the state a warp holds, for a head's key size.
static int gla_rows(int dim) { return dim <= 64 ? 8 : (dim <= 256 ? 16 : 32); }

VIPERA_API int vipera_gla_shares(int dim) { return (dim + gla_rows(dim) - 1) / gla_rows(dim); }

VIPERA_API int vipera_gla(const GlaParams* params, int out_dtype, void* stream) {
  GlaParams p = *params;
  if (p.num_tokens <= 0 || p.num_entries <= 0) return VIPERA_OK;
  if (p.heads <= 0 || p.dim <= 0 || p.dim > 512 || p.vdim <= 0) return VIPERA_BAD_SHAPE;
  if (!p.proj || !p.z || !p.log_alpha || !p.state || !p.entry_starts || !p.state_slots || !p.fresh || !p.partial || !p.norm_weight || !p.out)
    return VIPERA_BAD_ARGUMENT;
  const int rows = gla_rows(p.dim);
  p.shares = (p.dim + rows - 1) / rows;
  if (p.shares > kGlaMaxShares) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool chunked = p.num_jobs > 0 && p.chunk_state && p.chunk_decay;
  auto pass = [&](int mode) -> int {
    p.mode = mode;
    const int tiles = (p.vdim + 31) / 32;
    const int warps = std::min(tiles, kGlaWarps);
    dim3 grid(p.shares * ((tiles + kGlaWarps - 1) / kGlaWarps), p.heads, mode == 0 ? p.num_entries : p.num_jobs);
    if (mode == 1) {
      if (rows == 8) return vipera_launch(gla_scan_kernel<8, true>, grid, warps * 32, 0, s, p);
      if (rows == 16) return vipera_launch(gla_scan_kernel<16, true>, grid, warps * 32, 0, s, p);
      return vipera_launch(gla_scan_kernel<32, true>, grid, warps * 32, 0, s, p);
    }
    if (rows == 8) return vipera_launch(gla_scan_kernel<8, false>, grid, warps * 32, 0, s, p);
    if (rows == 16) return vipera_launch(gla_scan_kernel<16, false>, grid, warps * 32, 0, s, p);
    return vipera_launch(gla_scan_kernel<32, false>, grid, warps * 32, 0, s, p);
  };
  const size_t decays = static_cast<size_t>(p.num_tokens) * p.heads * p.dim;
  int status = vipera_launch(gla_decay_kernel, dim3(static_cast<unsigned>(std::min<size_t>((decays + 255) / 256, 4096))), 256, 0, s, p);
  if (status) return status;
  if (!chunked) status = pass(0);
  else {
    status = pass(1);
    if (!status) {
      const size_t width = static_cast<size_t>(p.heads) * p.dim * p.vdim;
      status = vipera_launch(gla_chunk_starts_kernel, dim3(static_cast<unsigned>((width + 255) / 256), p.num_entries), 256, 0, s, p);
    }
    if (!status) status = pass(3);
  }
  if (status) return status;
  const int items = p.num_tokens * p.heads;
  if (out_dtype == VIPERA_BF16) return vipera_launch(gla_finish_kernel<__nv_bfloat16>, (items + 3) / 4, 128, 0, s, p);
  if (out_dtype == VIPERA_F32) return vipera_launch(gla_finish_kernel<float>, (items + 3) / 4, 128, 0, s, p);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_gla_params_size() { return static_cast<int>(sizeof(GlaParams)); }
