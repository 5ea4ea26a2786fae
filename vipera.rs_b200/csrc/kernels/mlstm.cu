// The matrix-memory cell of xLSTM (mLSTM) over a step's entries: portions of prompts in chunks,
// single decode tokens one by one, both from the state that earlier steps left.
//
// The cell, per head, with a matrix S [d, dv], a vector n [d] and a running maximum m:
//   li = cap tanh(i / cap),  lf = logsigmoid(cap tanh(f / cap))        (log gates, capped)
//   m' = max(lf + m, li)
//   S' = exp(lf + m - m') S + exp(li - m') k v^T,   n' likewise with k alone
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + denom_eps),  q scaled by q_scale
// S, n and m start at `initial_max`-free zeros (m at 0) and live in 32-bit floats, one row per
// state slot: [S: heads * d * dv | n: heads * d | m: heads].
//
// A chunk of L tokens is computed at once.  With b_t the sum of lf over the chunk's tokens up
// to t, a_s = li_s - b_s and M_t = max(m_0, max_{s<=t} a_s), one has m_t = b_t + M_t and
//   S_t^T q_t = exp(m_0 - M_t) S_0^T q_t + sum_{s<=t} exp(a_s - M_t) (q_t . k_s) v_s
//   n_t . q_t = exp(m_0 - M_t) n_0 . q_t + sum_{s<=t} exp(a_s - M_t) (q_t . k_s)
//   S_L = exp(m_0 - M_L) S_0 + sum_s exp(a_s - M_L) k_s v_s^T
// Every exponent is at most 0.  All of it is 32-bit arithmetic on the CUDA cores; q, k, v and
// the gates' pre-activations come from one product (the caller's) as 32-bit values.
//
// A block owns (value-column tile, head, entry) and walks the entry's tokens chunk by chunk with
// its tile of S in shared memory.  n and m do not depend on the value columns: every tile
// computes them, tile 0 leaves the new ones in a scratch row, and the finishing kernel, which
// runs after all tiles have read the old ones, puts them into the state.  The finishing kernel
// divides each head's output by its root mean square, scales it, and gates it with
// sigmoid(g).
#include "common.cuh"

constexpr int kChunk = 32;      // tokens of a chunk
constexpr int kThreads = 256;

struct MlstmParams {
  const float* proj;        // [tokens, proj_width]: q | k | v | g | i | f (offsets below)
  int proj_width;
  int q_off, k_off, v_off, g_off, i_off, f_off;
  int heads, dim, vdim;
  int tile;                 // value columns per block
  int num_entries;
  float q_scale, gate_cap, denom_eps;
  const int* entry_starts;  // [entries + 1]
  const int* state_slots;   // [entries]
  const int* fresh;         // [entries] 1: the state starts anew
  float* state;             // [slots, state_stride]
  long long state_stride;
  float* o_raw;             // [tokens, heads, vdim] the cell's output before the head norm
  float* nm_scratch;        // [entries, heads, dim + 1] new n and m of each entry
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float capped(float x, float cap) { return cap * tanhf(x / cap); }

// ---------------------------------------------------------------------------------------
// portions: chunk by chunk
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
mlstm_chunk_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int d = p.dim, dv = p.vdim, TW = p.tile;
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * TW;
  const int cols = min(TW, dv - c0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = p.entry_starts[e], count = p.entry_starts[e + 1] - t0;
  if (count <= 0) return;
  const int dp = d + 1;                       // padded row of Q and K
  float* Qs = smem;                           // [kChunk][dp]
  float* Ks = Qs + kChunk * dp;               // [kChunk][dp]
  float* Vs = Ks + kChunk * dp;               // [kChunk][TW]
  float* Ws = Vs + kChunk * TW;               // [kChunk][kChunk + 1]
  float* Ss = Ws + kChunk * (kChunk + 1);     // [d][TW]
  float* ns = Ss + d * TW;                    // [d]
  float* av = ns + d;                         // [kChunk] a_s
  float* Mv = av + kChunk;                    // [kChunk] M_t
  float* bv = Mv + kChunk;                    // [kChunk] b_t
  float* den = bv + kChunk;                   // [kChunk]
  float* scal = den + kChunk;                 // [0] = running m

  float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
  float* S_state = state + static_cast<size_t>(h) * d * dv;
  float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
  float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
  const bool fresh = p.fresh[e] != 0;
  for (int item = tid; item < d * TW; item += kThreads) {
    const int dd = item / TW, c = item % TW;
    Ss[item] = (!fresh && c < cols) ? S_state[static_cast<size_t>(dd) * dv + c0 + c] : 0.0f;
  }
  for (int dd = tid; dd < d; dd += kThreads) ns[dd] = fresh ? 0.0f : n_state[dd];
  if (tid == 0) scal[0] = fresh ? 0.0f : m_state[0];

  for (int start = 0; start < count; start += kChunk) {
    const int len = min(kChunk, count - start);
    const float* rows = p.proj + static_cast<size_t>(t0 + start) * p.proj_width;
    __syncthreads();   // the chunk before is done with Q, K, V; S, n and m are in place
    for (int item = tid; item < kChunk * d; item += kThreads) {
      const int t = item / d, dd = item % d;
      float q = 0.0f, k = 0.0f;
      if (t < len) {
        const float* row = rows + static_cast<size_t>(t) * p.proj_width;
        q = row[p.q_off + h * d + dd] * p.q_scale;
        k = row[p.k_off + h * d + dd];
      }
      Qs[t * dp + dd] = q;
      Ks[t * dp + dd] = k;
    }
    for (int item = tid; item < kChunk * TW; item += kThreads) {
      const int t = item / TW, c = item % TW;
      Vs[item] = (t < len && c < cols) ? rows[static_cast<size_t>(t) * p.proj_width + p.v_off + h * dv + c0 + c] : 0.0f;
    }
    if (warp == 0) {
      // the gates of the chunk: one lane a token, sums and maxima along the lanes
      const float m0 = scal[0];
      float li = 0.0f, lf = 0.0f;
      if (lane < len) {
        const float* row = rows + static_cast<size_t>(lane) * p.proj_width;
        li = capped(row[p.i_off + h], p.gate_cap);
        lf = log_sigmoid(capped(row[p.f_off + h], p.gate_cap));
      }
      float b = lf;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, b, offset);
        if (lane >= offset) b += other;
      }
      const float a = lane < len ? li - b : -INFINITY;
      float top = a;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, top, offset);
        if (lane >= offset) top = fmaxf(top, other);
      }
      av[lane] = a;
      Mv[lane] = fmaxf(m0, top);
      bv[lane] = b;
    }
    __syncthreads();
    // W[t][s] = (q_t . k_s) exp(a_s - M_t) for s <= t
    {
      const int t = tid >> 3;
      float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const float* qrow = Qs + t * dp;
      for (int dd = 0; dd < d; ++dd) {
        const float q = qrow[dd];
#pragma unroll
        for (int j = 0; j < 4; ++j) dot[j] = fmaf(q, Ks[((tid & 7) + 8 * j) * dp + dd], dot[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int s = (tid & 7) + 8 * j;
        Ws[t * (kChunk + 1) + s] = (s <= t && t < len) ? dot[j] * expf(av[s] - Mv[t]) : 0.0f;
      }
    }
    __syncthreads();
    // denominators: one warp four rows
    {
      const float m0 = scal[0];
      for (int t = warp; t < kChunk; t += kThreads / 32) {
        float sum = Ws[t * (kChunk + 1) + lane];
        float qn = 0.0f;
        for (int dd = lane; dd < d; dd += 32) qn = fmaf(Qs[t * dp + dd], ns[dd], qn);
        sum = warp_sum(sum);
        qn = warp_sum(qn);
        if (lane == 0) {
          const float total = sum + expf(m0 - Mv[t]) * qn;
          den[t] = fmaxf(fabsf(total), expf(-(bv[t] + Mv[t]))) + p.denom_eps;
        }
      }
    }
    __syncthreads();
    // outputs: a thread one column, eight rows
    if (TW * 4 <= kThreads || tid < TW * (kThreads / TW)) {
      const int c = tid % TW, group = tid / TW, groups = kThreads / TW;
      const float m0 = scal[0];
      for (int tb = group; tb < kChunk; tb += groups * 8) {
        float inter[8], intra[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) inter[j] = intra[j] = 0.0f;
        for (int dd = 0; dd < d; ++dd) {
          const float s = Ss[dd * TW + c];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = tb + j * groups;
            if (t < kChunk) inter[j] = fmaf(Qs[t * dp + dd], s, inter[j]);
          }
        }
        for (int s = 0; s < len; ++s) {
          const float v = Vs[s * TW + c];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = tb + j * groups;
            if (t < kChunk) intra[j] = fmaf(Ws[t * (kChunk + 1) + s], v, intra[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = tb + j * groups;
          if (t < len && c < cols) {
            const float value = (intra[j] + expf(m0 - Mv[t]) * inter[j]) / den[t];
            p.o_raw[(static_cast<size_t>(t0 + start + t) * p.heads + h) * dv + c0 + c] = value;
          }
        }
      }
    }
    __syncthreads();
    // the state at the chunk's end
    const float M_last = Mv[len - 1];
    const float keep = expf(scal[0] - M_last);
    for (int item = tid; item < kChunk * TW; item += kThreads) {
      const int s = item / TW;
      Vs[item] *= s < len ? expf(av[s] - M_last) : 0.0f;
    }
    __syncthreads();
    {
      const int c = tid % TW, group = tid / TW, groups = kThreads / TW;
      for (int db = group; db < d; db += groups * 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int s = 0; s < len; ++s) {
          const float v = Vs[s * TW + c];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int dd = db + j * groups;
            if (dd < d) acc[j] = fmaf(Ks[s * dp + dd], v, acc[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int dd = db + j * groups;
          if (dd < d) Ss[dd * TW + c] = keep * Ss[dd * TW + c] + acc[j];
        }
      }
    }
    for (int dd = tid; dd < d; dd += kThreads) {
      float acc = 0.0f;
      for (int s = 0; s < len; ++s) acc = fmaf(expf(av[s] - M_last), Ks[s * dp + dd], acc);
      ns[dd] = keep * ns[dd] + acc;
    }
    __syncthreads();
    if (tid == 0) scal[0] = bv[len - 1] + M_last;
  }
  __syncthreads();
  for (int item = tid; item < d * TW; item += kThreads) {
    const int dd = item / TW, c = item % TW;
    if (c < cols) S_state[static_cast<size_t>(dd) * dv + c0 + c] = Ss[item];
  }
  if (blockIdx.x == 0) {
    float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
    for (int dd = tid; dd < d; dd += kThreads) scratch[dd] = ns[dd];
    if (tid == 0) scratch[d] = scal[0];
  }
}

// ---------------------------------------------------------------------------------------
// single tokens: one pass over the state
// ---------------------------------------------------------------------------------------
// Every entry brings one token.  A block owns (value-column tile of 64, head, entry): a thread a
// column and a quarter of the rows; the state is read and written once.
constexpr int kDecodeTile = 64;

__global__ void __launch_bounds__(kThreads)
mlstm_decode_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int d = p.dim, dv = p.vdim;
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * kDecodeTile;
  const int tid = threadIdx.x;
  const int t0 = p.entry_starts[e];
  if (p.entry_starts[e + 1] - t0 != 1) return;
  float* qs = smem;             // [d]
  float* ks = qs + d;           // [d]
  float* part = ks + d;         // [4][64]
  float* red = part + 4 * kDecodeTile;  // [32] reduction scratch
  float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
  float* S_state = state + static_cast<size_t>(h) * d * dv;
  float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
  float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
  const bool fresh = p.fresh[e] != 0;
  const float* row = p.proj + static_cast<size_t>(t0) * p.proj_width;
  for (int dd = tid; dd < d; dd += kThreads) {
    qs[dd] = row[p.q_off + h * d + dd] * p.q_scale;
    ks[dd] = row[p.k_off + h * d + dd];
  }
  const float li = capped(row[p.i_off + h], p.gate_cap);
  const float lf = log_sigmoid(capped(row[p.f_off + h], p.gate_cap));
  const float m_old = fresh ? 0.0f : m_state[0];
  const float m_new = fmaxf(lf + m_old, li);
  const float keep = fresh ? 0.0f : expf(lf + m_old - m_new);
  const float take = expf(li - m_new);
  __syncthreads();
  // n' . q over the block, and n' into the scratch by tile 0
  float qn = 0.0f;
  float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
  for (int dd = tid; dd < d; dd += kThreads) {
    const float n_new = (fresh ? 0.0f : keep * n_state[dd]) + take * ks[dd];
    qn = fmaf(n_new, qs[dd], qn);
    if (blockIdx.x == 0) scratch[dd] = n_new;
  }
  if (blockIdx.x == 0 && tid == 0) scratch[d] = m_new;
  qn = block_sum(qn, red);
  const float denominator = fmaxf(fabsf(qn), expf(-m_new)) + p.denom_eps;
  const int c = tid & (kDecodeTile - 1), group = tid / kDecodeTile;   // 4 groups of rows
  const bool live = c0 + c < dv;
  float acc = 0.0f;
  if (live) {
    const float v = row[p.v_off + h * dv + c0 + c] * take;
    float* column = S_state + c0 + c;
    int dd = group;
    for (; dd + 28 < d; dd += 32) {
      float s[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = fresh ? 0.0f : column[static_cast<size_t>(dd + 4 * j) * dv];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j] = fmaf(ks[dd + 4 * j], v, keep * s[j]);
        column[static_cast<size_t>(dd + 4 * j) * dv] = s[j];
        acc = fmaf(s[j], qs[dd + 4 * j], acc);
      }
    }
    for (; dd < d; dd += 4) {
      float s = fresh ? 0.0f : column[static_cast<size_t>(dd) * dv];
      s = fmaf(ks[dd], v, keep * s);
      column[static_cast<size_t>(dd) * dv] = s;
      acc = fmaf(s, qs[dd], acc);
    }
  }
  part[group * kDecodeTile + c] = acc;
  __syncthreads();
  if (tid < kDecodeTile && c0 + tid < dv) {
    const float total = part[tid] + part[kDecodeTile + tid] + part[2 * kDecodeTile + tid] + part[3 * kDecodeTile + tid];
    p.o_raw[(static_cast<size_t>(t0) * p.heads + h) * dv + c0 + tid] = total / denominator;
  }
}

// ---------------------------------------------------------------------------------------
// the ending: head norm, scale, output gate; and the new n and m into the state
// ---------------------------------------------------------------------------------------
// One warp per (token, head).  out[t, h*dv + c] = o / rms(o) * weight[h*dv + c] * sigmoid(g[t, h*dv + c]).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_finish_kernel(const MlstmParams p, const float* __restrict__ weight, float eps, T* __restrict__ out,
                    const int* __restrict__ token_entry) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
  if (h >= p.heads) return;
  const int dv = p.vdim, d = p.dim;
  const float* o = p.o_raw + (static_cast<size_t>(t) * p.heads + h) * dv;
  float squares = 0.0f;
  for (int c = lane; c < dv; c += 32) squares = fmaf(o[c], o[c], squares);
  squares = warp_sum(squares);
  const float inverse = rsqrtf(squares / static_cast<float>(dv) + eps);
  const float* gate = p.proj + static_cast<size_t>(t) * p.proj_width + p.g_off + h * dv;
  const float* w = weight + h * dv;
  T* dst = out + static_cast<size_t>(t) * p.heads * dv + h * dv;
  for (int c = lane; c < dv; c += 32) {
    const float g = 1.0f / (1.0f + expf(-gate[c]));
    dst[c] = from_float<T>(o[c] * inverse * w[c] * g);
  }
  const int e = token_entry[t];
  if (t == p.entry_starts[e + 1] - 1) {
    float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
    float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
    float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
    const float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
    for (int dd = lane; dd < d; dd += 32) n_state[dd] = scratch[dd];
    if (lane == 0) m_state[0] = scratch[d];
  }
}

static size_t chunk_shared_bytes(int d, int tile) {
  return sizeof(float) * (2 * kChunk * (d + 1) + kChunk * tile + kChunk * (kChunk + 1) + static_cast<size_t>(d) * tile +
                          d + 4 * kChunk + 4);
}

// The value columns a block of the chunk kernel takes for these sizes (0: the sizes are refused).
VIPERA_API int vipera_mlstm_tile(int dim, int vdim) {
  if (dim <= 0 || vdim <= 0) return 0;
  for (int tile = 64; tile >= 8; tile >>= 1) {
    if (tile > 8 && tile >= 2 * vdim) continue;          // narrower heads take narrower tiles
    if (chunk_shared_bytes(dim, tile) <= 200 * 1024) return tile;
  }
  return 0;
}

VIPERA_API int vipera_mlstm_params_size() { return static_cast<int>(sizeof(MlstmParams)); }

// Floats of one state row: S, n and m of every head, rounded up to a multiple of four.
VIPERA_API long long vipera_mlstm_state_floats(int heads, int dim, int vdim) {
  const long long raw = static_cast<long long>(heads) * (static_cast<long long>(dim) * vdim + dim + 1);
  return (raw + 3) / 4 * 4;
}

// Runs the cell over a step: `single` != 0 promises that every entry brings one token.
// out is [tokens, heads * vdim] in `out_dtype`.
VIPERA_API int vipera_mlstm(const MlstmParams* params, int num_tokens, int single, const float* norm_weight,
                            float norm_eps, void* out, int out_dtype, const int* token_entry, void* stream) {
  MlstmParams p = *params;
  if (num_tokens <= 0 || p.num_entries <= 0) return VIPERA_OK;
  if (p.heads <= 0 || p.dim <= 0 || p.vdim <= 0 || !(p.gate_cap > 0.0f)) return VIPERA_BAD_SHAPE;
  if (!p.proj || !p.state || !p.o_raw || !p.nm_scratch || !p.entry_starts || !p.state_slots || !p.fresh || !out ||
      !token_entry || !norm_weight)
    return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status;
  if (single) {
    dim3 grid((p.vdim + kDecodeTile - 1) / kDecodeTile, p.heads, p.num_entries);
    const size_t shared = sizeof(float) * (2 * p.dim + 4 * kDecodeTile + 32);
    if (shared > 200 * 1024) return VIPERA_BAD_SHAPE;
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(mlstm_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    status = vipera_launch(mlstm_decode_kernel, grid, kThreads, shared, s, p);
  } else {
    p.tile = vipera_mlstm_tile(p.dim, p.vdim);
    if (p.tile == 0) return VIPERA_BAD_SHAPE;
    dim3 grid((p.vdim + p.tile - 1) / p.tile, p.heads, p.num_entries);
    const size_t shared = chunk_shared_bytes(p.dim, p.tile);
    static size_t allowed = 0;
    if (shared > 48 * 1024 && shared > allowed) {
      cudaError_t error = cudaFuncSetAttribute(mlstm_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(shared));
      if (error != cudaSuccess) return static_cast<int>(error);
      allowed = shared;
    }
    status = vipera_launch(mlstm_chunk_kernel, grid, kThreads, shared, s, p);
  }
  if (status != 0) return status;
  dim3 grid(num_tokens, (p.heads + 3) / 4);
  if (out_dtype == VIPERA_F32)
    return vipera_launch(mlstm_finish_kernel<float>, grid, 128, 0, s, p, norm_weight, norm_eps, static_cast<float*>(out),
                         token_entry);
  if (out_dtype == VIPERA_BF16)
    return vipera_launch(mlstm_finish_kernel<__nv_bfloat16>, grid, 128, 0, s, p, norm_weight, norm_eps,
                         static_cast<__nv_bfloat16*>(out), token_entry);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API const char* vipera_mlstm_status_text(int status) { return vipera_status_text(status); }
