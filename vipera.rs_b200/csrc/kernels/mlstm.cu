// The matrix-memory cell of xLSTM (mLSTM) over a step's entries: portions of prompts in chunks,
// single decode tokens one by one, both from the state that earlier steps left.
//
// The cell, per head, with a matrix S [d, dv], a vector n [d] and a running maximum m:
//   li = cap tanh(i / cap),  lf = logsigmoid(cap tanh(f / cap))        (log gates, capped)
//   m' = max(lf + m, li)
//   S' = exp(lf + m - m') S + exp(li - m') k v^T,   n' likewise with k alone
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + denom_eps),  q scaled by q_scale
// S, n and m start at zero (m at 0, not at minus infinity) and live in 32-bit floats, one row per
// state slot: [S: heads * d * dv | n: heads * d | m: heads].
//
// A chunk of L tokens is computed at once.  With b_t the sum of lf over the chunk's tokens up
// to t, a_s = li_s - b_s and M_t = max(m_0, max_{s<=t} a_s), one has m_t = b_t + M_t and
//   S_t^T q_t = exp(m_0 - M_t) S_0^T q_t + sum_{s<=t} exp(a_s - M_t) (q_t . k_s) v_s
//   n_t . q_t = exp(m_0 - M_t) n_0 . q_t + sum_{s<=t} exp(a_s - M_t) (q_t . k_s)
//   S_L = exp(m_0 - M_L) S_0 + sum_s exp(a_s - M_L) k_s v_s^T
// Every exponent is at most 0.  q, k, v and the gates' pre-activations come from one product (the
// caller's) as 32-bit values.  The first kernel below is that form in 32-bit arithmetic on the CUDA
// cores (the 32-bit run, and sizes the others do not take); further down the same on the tensor
// cores for bfloat16 runs, walking an entry's chunks or computing all chunks of a step at once.
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
  // the form that computes all chunks of a step at once (see mlstm_parts_kernel)
  float* chunk_state;       // [jobs, heads, dim, vdim] a chunk's own sum, then the state at its start
  float* chunk_n;           // [jobs, heads, dim]       the same for n
  float* chunk_aux;         // [jobs, heads, 4]         the chunk's largest a_s, its sum of log forget gates, m at its start
  int max_jobs;
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
// portions on the tensor cores (bfloat16 runs; q/k sizes 64, 128 and 256)
// ---------------------------------------------------------------------------------------
// The same chunked form with chunks of 64 tokens and its four products as mma.sync m16n8k16
// (bfloat16 operands, 32-bit accumulators): scores Q K^T, the weighted values W V, the read of
// the old state Q S, and the update K^T (w V).  A block of eight warps owns (64 value columns,
// head, entry).  Its tile of S lives in the accumulators of the update product from the first
// chunk to the last, in 32-bit, and is never rounded; a bfloat16 copy, transposed, is laid into
// shared memory after every update for the read product.  Gates, maxima, weights, row sums and
// denominators are 32-bit arithmetic as in the kernel above; q, k, v and the weights enter the
// products as bfloat16.  Every operand lies in shared memory with the product's inner index
// contiguous (K and V also transposed), rows padded by 16 bytes, so that a fragment is four
// 32-bit loads without bank conflicts.
constexpr int kTcChunk = 64, kTcTile = 64, kTcThreads = 256;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }
// Four neighbouring 32-bit values: one 16-byte load where the caller knows the address to be aligned.
__device__ __forceinline__ float4 load4(const float* at, bool wide) {
  if (wide) return *reinterpret_cast<const float4*>(at);
  return make_float4(at[0], at[1], at[2], at[3]);
}
// Whether every q and k row of the product's result starts on 16 bytes.
__device__ __forceinline__ bool rows_wide(const MlstmParams& p) {
  return ((reinterpret_cast<uintptr_t>(p.proj) & 15) == 0) && p.proj_width % 4 == 0 && p.q_off % 4 == 0 && p.k_off % 4 == 0 &&
         p.dim % 4 == 0;
}
// A fragment (16 x 16) of a row-major array with `stride` elements a row, at (row0, k0).
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __nv_bfloat16* base, int stride, int row0, int k0, int g, int tq) {
  const __nv_bfloat16* at = base + (row0 + g) * stride + k0 + 2 * tq;
  a[0] = ld32(at);
  a[1] = ld32(at + 8 * stride);
  a[2] = ld32(at + 8);
  a[3] = ld32(at + 8 * stride + 8);
}

template <int D>
struct TcLayout {
  static constexpr int kQS = D + 8;           // elements a row of Q, K and S^T
  static constexpr int kLS = kTcChunk + 8;    // elements a row of K^T, V^T and W
  static constexpr size_t kHalves = 2 * kTcChunk * kQS + D * kLS + kTcTile * kLS + kTcChunk * kLS + kTcTile * kQS;
  static constexpr size_t kFloats = D + 9 * kTcChunk + 8;
  static constexpr size_t kBytes = kHalves * 2 + kFloats * 4;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads)
mlstm_chunk_tc_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int L = kTcChunk, TW = kTcTile, QS = TcLayout<D>::kQS, LS = TcLayout<D>::kLS;
  // who owns which part of S: WM x WN warps, each MT x NT tiles of 16 x 8
  constexpr int WM = D >= 128 ? 8 : 4, WN = 8 / WM, MT = D / 16 / WM, NT = 8 / WN;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(raw);   // [L][QS]
  __nv_bfloat16* Ks = Qs + L * QS;                             // [L][QS]
  __nv_bfloat16* Kt = Ks + L * QS;                             // [D][LS]   K transposed
  __nv_bfloat16* Vt = Kt + D * LS;                             // [TW][LS]  V transposed
  __nv_bfloat16* Ws = Vt + TW * LS;                            // [L][LS]   weights of the chunk
  __nv_bfloat16* St = Ws + L * LS;                             // [TW][QS]  S transposed, bfloat16
  float* ns = reinterpret_cast<float*>(St + TW * QS);          // [D]
  float* av = ns + D;        // [L] a_s
  float* Mv = av + L;        // [L] M_t
  float* bv = Mv + L;        // [L] b_t
  float* lis = bv + L;       // [L] log input gates
  float* lfs = lis + L;      // [L] log forget gates
  float* rs = lfs + L;       // [2][L] halves of the weights' row sums
  float* qn = rs + 2 * L;    // [L] q_t . n_0
  float* we = qn + L;        // [L] exp(a_s - M_L)
  float* scal = we + L;      // [0] the running m

  const int d = D, dv = p.vdim;
  const bool wide = rows_wide(p);
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * TW;
  const int cols = min(TW, dv - c0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int t0 = p.entry_starts[e], count = p.entry_starts[e + 1] - t0;
  if (count <= 0) return;
  const int rm = warp & 3, cn = warp >> 2;      // the scores' and outputs' tile: rows rm*16.., columns cn*32..
  const int sm = warp % WM, sn = warp / WM;     // the state's tile

  float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
  float* S_state = state + static_cast<size_t>(h) * d * dv;
  float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
  float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
  const bool fresh = p.fresh[e] != 0;

  float S[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int dd = (sm * MT + mt) * 16 + g + 8 * (i >> 1), c = (sn * NT + nt) * 8 + 2 * tq + (i & 1);
        const float value = (!fresh && c < cols) ? S_state[static_cast<size_t>(dd) * dv + c0 + c] : 0.0f;
        S[mt][nt][i] = value;
        St[c * QS + dd] = __float2bfloat16_rn(value);
      }
  for (int dd = tid; dd < d; dd += kTcThreads) ns[dd] = fresh ? 0.0f : n_state[dd];
  if (tid == 0) scal[0] = fresh ? 0.0f : m_state[0];

  for (int start = 0; start < count; start += L) {
    const int len = min(L, count - start);
    const float* rows = p.proj + static_cast<size_t>(t0 + start) * p.proj_width;
    __syncthreads();   // the chunk before is done with its tiles; S^T, n and m are in place
    for (int item = tid; item < L * (D / 4); item += kTcThreads) {
      const int t = item / (D / 4), dd = (item % (D / 4)) * 4;
      float4 q = make_float4(0.0f, 0.0f, 0.0f, 0.0f), k = q;
      if (t < len) {
        const float* row = rows + static_cast<size_t>(t) * p.proj_width;
        q = load4(row + p.q_off + h * d + dd, wide);
        k = load4(row + p.k_off + h * d + dd, wide);
      }
      const __nv_bfloat162 k01 = __floats2bfloat162_rn(k.x, k.y), k23 = __floats2bfloat162_rn(k.z, k.w);
      *reinterpret_cast<__nv_bfloat162*>(Qs + t * QS + dd) = __floats2bfloat162_rn(q.x * p.q_scale, q.y * p.q_scale);
      *reinterpret_cast<__nv_bfloat162*>(Qs + t * QS + dd + 2) = __floats2bfloat162_rn(q.z * p.q_scale, q.w * p.q_scale);
      *reinterpret_cast<__nv_bfloat162*>(Ks + t * QS + dd) = k01;
      *reinterpret_cast<__nv_bfloat162*>(Ks + t * QS + dd + 2) = k23;
      Kt[dd * LS + t] = k01.x;
      Kt[(dd + 1) * LS + t] = k01.y;
      Kt[(dd + 2) * LS + t] = k23.x;
      Kt[(dd + 3) * LS + t] = k23.y;
    }
    for (int item = tid; item < L * TW; item += kTcThreads) {
      const int t = item / TW, c = item % TW;
      const float v = (t < len && c < cols) ? rows[static_cast<size_t>(t) * p.proj_width + p.v_off + h * dv + c0 + c] : 0.0f;
      Vt[c * LS + t] = __float2bfloat16_rn(v);
    }
    if (tid < L) {
      float li = 0.0f, lf = 0.0f;
      if (tid < len) {
        const float* row = rows + static_cast<size_t>(tid) * p.proj_width;
        li = capped(row[p.i_off + h], p.gate_cap);
        lf = log_sigmoid(capped(row[p.f_off + h], p.gate_cap));
      }
      lis[tid] = li;
      lfs[tid] = lf;
    }
    __syncthreads();
    if (tid == 0) {
      float b = 0.0f, top = -INFINITY;
      const float m0 = scal[0];
      for (int t = 0; t < L; ++t) {
        b += lfs[t];
        const float a = t < len ? lis[t] - b : -INFINITY;
        top = fmaxf(top, a);
        av[t] = a;
        bv[t] = b;
        Mv[t] = fmaxf(m0, top);
      }
    }
    __syncthreads();
    const float m0 = scal[0];
    // scores and weights: rows rm*16 .., keys cn*32 ..
    {
      float G[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) G[j][i] = 0.0f;
#pragma unroll 4
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        load_a(a, Qs, QS, rm * 16, kk * 16, g, tq);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat16* at = Ks + (cn * 32 + j * 8 + g) * QS + kk * 16 + 2 * tq;
          mma_bf16(G[j], a, ld32(at), ld32(at + 8));
        }
      }
      float sums[2] = {0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int t = rm * 16 + g + 8 * r, s0 = cn * 32 + j * 8 + 2 * tq;
          float w[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int sk = s0 + i;
            w[i] = (sk <= t && t < len) ? G[j][2 * r + i] * expf(av[sk] - Mv[t]) : 0.0f;
            sums[r] += w[i];
          }
          *reinterpret_cast<__nv_bfloat162*>(Ws + t * LS + s0) = __floats2bfloat162_rn(w[0], w[1]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sums[r] += __shfl_xor_sync(0xffffffffu, sums[r], 1);
        sums[r] += __shfl_xor_sync(0xffffffffu, sums[r], 2);
        if (tq == 0) rs[cn * L + rm * 16 + g + 8 * r] = sums[r];
      }
    }
    // q_t . n_0: four threads a row
    {
      const int t = tid >> 2, part = tid & 3;
      float sum = 0.0f;
      for (int dd = part; dd < D; dd += 4) sum = fmaf(__bfloat162float(Qs[t * QS + dd]), ns[dd], sum);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (part == 0) qn[t] = sum;
    }
    __syncthreads();
    // outputs: the old state's share first, then the chunk's own
    {
      float O[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) O[j][i] = 0.0f;
#pragma unroll 4
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        load_a(a, Qs, QS, rm * 16, kk * 16, g, tq);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat16* at = St + (cn * 32 + j * 8 + g) * QS + kk * 16 + 2 * tq;
          mma_bf16(O[j], a, ld32(at), ld32(at + 8));
        }
      }
      float inter[2], denominator[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int t = rm * 16 + g + 8 * r;
        inter[r] = expf(m0 - Mv[t]);
        const float total = rs[t] + rs[L + t] + inter[r] * qn[t];
        denominator[r] = fmaxf(fabsf(total), expf(-(bv[t] + Mv[t]))) + p.denom_eps;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) O[j][i] *= inter[i >> 1];
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk) {
        uint32_t a[4];
        load_a(a, Ws, LS, rm * 16, kk * 16, g, tq);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat16* at = Vt + (cn * 32 + j * 8 + g) * LS + kk * 16 + 2 * tq;
          mma_bf16(O[j], a, ld32(at), ld32(at + 8));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = rm * 16 + g + 8 * (i >> 1), c = cn * 32 + j * 8 + 2 * tq + (i & 1);
          if (t < len && c < cols)
            p.o_raw[(static_cast<size_t>(t0 + start + t) * p.heads + h) * dv + c0 + c] = O[j][i] / denominator[i >> 1];
        }
    }
    __syncthreads();
    // the state at the chunk's end: S = exp(m_0 - M_L) S + K^T (w V)
    const float M_last = Mv[len - 1];
    const float keep = expf(m0 - M_last);
    if (tid < L) we[tid] = tid < len ? expf(av[tid] - M_last) : 0.0f;
    for (int item = tid; item < L * TW; item += kTcThreads) {
      const int c = item / L, t = item % L;
      const float w = t < len ? expf(av[t] - M_last) : 0.0f;
      Vt[c * LS + t] = __float2bfloat16_rn(__bfloat162float(Vt[c * LS + t]) * w);
    }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) S[mt][nt][i] *= keep;
#pragma unroll
    for (int kk = 0; kk < L / 16; ++kk) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        load_a(a, Kt, LS, (sm * MT + mt) * 16, kk * 16, g, tq);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const __nv_bfloat16* at = Vt + ((sn * NT + nt) * 8 + g) * LS + kk * 16 + 2 * tq;
          mma_bf16(S[mt][nt], a, ld32(at), ld32(at + 8));
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int dd = (sm * MT + mt) * 16 + g + 8 * (i >> 1), c = (sn * NT + nt) * 8 + 2 * tq + (i & 1);
          St[c * QS + dd] = __float2bfloat16_rn(S[mt][nt][i]);
        }
    for (int dd = tid; dd < d; dd += kTcThreads) {
      float acc = 0.0f;
      for (int t = 0; t < len; ++t) acc = fmaf(we[t], __bfloat162float(Kt[dd * LS + t]), acc);
      ns[dd] = keep * ns[dd] + acc;
    }
    if (tid == 0) scal[0] = bv[len - 1] + M_last;
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int dd = (sm * MT + mt) * 16 + g + 8 * (i >> 1), c = (sn * NT + nt) * 8 + 2 * tq + (i & 1);
        if (c < cols) S_state[static_cast<size_t>(dd) * dv + c0 + c] = S[mt][nt][i];
      }
  if (blockIdx.x == 0) {
    float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
    for (int dd = tid; dd < d; dd += kTcThreads) scratch[dd] = ns[dd];
    if (tid == 0) scratch[d] = scal[0];
  }
}

// ---------------------------------------------------------------------------------------
// portions on the tensor cores, all chunks at once
// ---------------------------------------------------------------------------------------
// The kernel above walks an entry's chunks one after another, so a long prompt keeps only
// (value tiles x heads) blocks busy.  Here the chunks of a step are jobs of their own, numbered
// entry by entry, and the work is cut in three:
//   1. mlstm_parts_kernel, a block per (value tile, head, job): the chunk's own contribution to
//      the state, U = sum_s exp(a_s - A) k_s v_s^T with A = max_s a_s, likewise u for n, and the
//      chunk's A and sum of log forget gates B;
//   2. mlstm_scan_kernel, elementwise over S with the chunks in order: M = max(m, A);
//      the state at the chunk's start takes U's place in memory; S = exp(m - M) S + exp(A - M) U;
//      m = B + M; at the end the new S goes into the state, n and m into the scratch row;
//   3. mlstm_outputs_kernel, a block per (value tile, head, job): scores, weights, row sums and
//      outputs of the chunk from the state, n and m at its start, exactly as in the kernel above.
// The sums are associated differently from the walking kernel's (U is summed before it meets
// S), which is 32-bit rounding only.
__device__ __forceinline__ bool find_job(const MlstmParams& p, int job, int* entry, int* chunk) {
  int remaining = job;
  for (int e = 0; e < p.num_entries; ++e) {
    const int count = p.entry_starts[e + 1] - p.entry_starts[e];
    const int chunks = (count + kTcChunk - 1) / kTcChunk;
    if (remaining < chunks) {
      *entry = e;
      *chunk = remaining;
      return true;
    }
    remaining -= chunks;
  }
  return false;
}

template <int D>
struct PartsLayout {
  static constexpr int kLS = kTcChunk + 8;
  static constexpr size_t kBytes = (static_cast<size_t>(D) * kLS + kTcTile * kLS) * 2 + (3 * kTcChunk + 8) * 4;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads)
mlstm_parts_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int L = kTcChunk, TW = kTcTile, LS = PartsLayout<D>::kLS;
  constexpr int WM = D >= 128 ? 8 : 4, WN = 8 / WM, MT = D / 16 / WM, NT = 8 / WN;
  int e, chunk;
  if (!find_job(p, blockIdx.z, &e, &chunk)) return;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(raw);   // [D][LS]
  __nv_bfloat16* Vt = Kt + D * LS;                             // [TW][LS]
  float* lis = reinterpret_cast<float*>(Vt + TW * LS);         // [L]
  float* lfs = lis + L;                                        // [L]
  float* we = lfs + L;                                         // [L] exp(a_s - A)
  float* scal = we + L;                                        // [0] A, [1] B
  const int d = D, dv = p.vdim;
  const bool wide = rows_wide(p);
  const int h = blockIdx.y, c0 = blockIdx.x * TW, job = blockIdx.z;
  const int cols = min(TW, dv - c0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int t0 = p.entry_starts[e], count = p.entry_starts[e + 1] - t0;
  const int start = chunk * L, len = min(L, count - start);
  const int sm = warp % WM, sn = warp / WM;
  const float* rows = p.proj + static_cast<size_t>(t0 + start) * p.proj_width;
  if (tid < L) {
    float li = 0.0f, lf = 0.0f;
    if (tid < len) {
      const float* row = rows + static_cast<size_t>(tid) * p.proj_width;
      li = capped(row[p.i_off + h], p.gate_cap);
      lf = log_sigmoid(capped(row[p.f_off + h], p.gate_cap));
    }
    lis[tid] = li;
    lfs[tid] = lf;
  }
  __syncthreads();
  if (warp == 0) {
    // a_s = li_s - b_s for two tokens a lane; the largest of them; the sum of the log forget gates
    float first = lfs[2 * lane], second = lfs[2 * lane + 1];
    float pair = first + second, before = pair;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const float other = __shfl_up_sync(0xffffffffu, before, offset);
      if (lane >= offset) before += other;
    }
    const float b0 = before - pair + first, b1 = before;          // inclusive sums at 2 lane and 2 lane + 1
    const float a0 = 2 * lane < len ? lis[2 * lane] - b0 : -INFINITY;
    const float a1 = 2 * lane + 1 < len ? lis[2 * lane + 1] - b1 : -INFINITY;
    const float top = warp_max(fmaxf(a0, a1));
    we[2 * lane] = 2 * lane < len ? expf(a0 - top) : 0.0f;
    we[2 * lane + 1] = 2 * lane + 1 < len ? expf(a1 - top) : 0.0f;
    const float total = __shfl_sync(0xffffffffu, before, 31);
    if (lane == 0) {
      scal[0] = top;
      scal[1] = total;
    }
  }
  __syncthreads();
  for (int item = tid; item < L * (D / 4); item += kTcThreads) {
    const int t = item / (D / 4), dd = (item % (D / 4)) * 4;
    float4 k = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < len) k = load4(rows + static_cast<size_t>(t) * p.proj_width + p.k_off + h * d + dd, wide);
    Kt[dd * LS + t] = __float2bfloat16_rn(k.x);
    Kt[(dd + 1) * LS + t] = __float2bfloat16_rn(k.y);
    Kt[(dd + 2) * LS + t] = __float2bfloat16_rn(k.z);
    Kt[(dd + 3) * LS + t] = __float2bfloat16_rn(k.w);
  }
  for (int item = tid; item < L * TW; item += kTcThreads) {
    const int t = item / TW, c = item % TW;
    const float v = (t < len && c < cols) ? rows[static_cast<size_t>(t) * p.proj_width + p.v_off + h * dv + c0 + c] : 0.0f;
    Vt[c * LS + t] = __float2bfloat16_rn(v * we[t]);
  }
  __syncthreads();
  float S[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) S[mt][nt][i] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < L / 16; ++kk) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint32_t a[4];
      load_a(a, Kt, LS, (sm * MT + mt) * 16, kk * 16, g, tq);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const __nv_bfloat16* at = Vt + ((sn * NT + nt) * 8 + g) * LS + kk * 16 + 2 * tq;
        mma_bf16(S[mt][nt], a, ld32(at), ld32(at + 8));
      }
    }
  }
  float* U = p.chunk_state + (static_cast<size_t>(job) * p.heads + h) * d * dv;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; i += 2) {
        const int dd = (sm * MT + mt) * 16 + g + 8 * (i >> 1), c = (sn * NT + nt) * 8 + 2 * tq;
        if (c + 1 < cols) *reinterpret_cast<float2*>(U + static_cast<size_t>(dd) * dv + c0 + c) = make_float2(S[mt][nt][i], S[mt][nt][i + 1]);
        else if (c < cols) U[static_cast<size_t>(dd) * dv + c0 + c] = S[mt][nt][i];
      }
  if (blockIdx.x == 0) {
    float* u = p.chunk_n + (static_cast<size_t>(job) * p.heads + h) * d;
    for (int dd = tid; dd < d; dd += kTcThreads) {
      float acc = 0.0f;
      for (int t = 0; t < len; ++t) acc = fmaf(we[t], __bfloat162float(Kt[dd * LS + t]), acc);
      u[dd] = acc;
    }
    if (tid == 0) {
      float* aux = p.chunk_aux + (static_cast<size_t>(job) * p.heads + h) * 4;
      aux[0] = scal[0];
      aux[1] = scal[1];
    }
  }
}

// grid: (parts of S, heads, entries); a thread four neighbouring values of S, the chunks in order.
__global__ void __launch_bounds__(256)
mlstm_scan_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.z, h = blockIdx.y;
  const int d = p.dim, dv = p.vdim;
  const int t0 = p.entry_starts[e], count = p.entry_starts[e + 1] - t0;
  if (count <= 0) return;
  const int chunks = (count + kTcChunk - 1) / kTcChunk;
  int job0 = 0;
  for (int other = 0; other < e; ++other)
    job0 += (p.entry_starts[other + 1] - p.entry_starts[other] + kTcChunk - 1) / kTcChunk;
  float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
  float* S_state = state + static_cast<size_t>(h) * d * dv;
  const float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
  const float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
  const bool fresh = p.fresh[e] != 0;
  const size_t index = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const size_t total = static_cast<size_t>(d) * dv;
  const size_t job_stride = static_cast<size_t>(p.heads) * total;
  float4 S = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  const bool live = index < total;
  if (live && !fresh) S = *reinterpret_cast<const float4*>(S_state + index);
  float m = fresh ? 0.0f : m_state[0];
  // n rides along in the first block: a thread a value
  const bool with_n = blockIdx.x == 0;
  float n[2] = {0.0f, 0.0f};
  if (with_n && !fresh)
    for (int i = 0; i < 2; ++i)
      if (threadIdx.x + 256 * i < d) n[i] = n_state[threadIdx.x + 256 * i];
  float* U = p.chunk_state + (static_cast<size_t>(job0) * p.heads + h) * total + index;
  for (int c0 = 0; c0 < chunks; c0 += 4) {
    float4 own[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (live && c0 + j < chunks) own[j] = *reinterpret_cast<const float4*>(U + (c0 + j) * job_stride);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c0 + j >= chunks) break;
      const int job = job0 + c0 + j;
      float* aux = p.chunk_aux + (static_cast<size_t>(job) * p.heads + h) * 4;
      const float A = aux[0], B = aux[1];
      const float M = fmaxf(m, A);
      const float keep = expf(m - M), take = expf(A - M);
      if (live) {
        *reinterpret_cast<float4*>(U + (c0 + j) * job_stride) = S;   // the state at the chunk's start
        S = make_float4(keep * S.x + take * own[j].x, keep * S.y + take * own[j].y, keep * S.z + take * own[j].z,
                        keep * S.w + take * own[j].w);
      }
      if (with_n) {
        float* u = p.chunk_n + (static_cast<size_t>(job) * p.heads + h) * d;
        for (int i = 0; i < 2; ++i) {
          const int dd = threadIdx.x + 256 * i;
          if (dd < d) {
            const float mine = u[dd];
            u[dd] = n[i];
            n[i] = keep * n[i] + take * mine;
          }
        }
        if (threadIdx.x == 0) aux[2] = m;
      }
      m = B + M;
    }
  }
  if (live) *reinterpret_cast<float4*>(S_state + index) = S;
  if (with_n) {
    float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
    for (int i = 0; i < 2; ++i)
      if (threadIdx.x + 256 * i < d) scratch[threadIdx.x + 256 * i] = n[i];
    if (threadIdx.x == 0) scratch[d] = m;
  }
}

template <int D>
struct OutputsLayout {
  static constexpr int kQS = D + 8, kLS = kTcChunk + 8;
  // (S^T takes K's place once the scores are done: two blocks fit an SM at the largest size)
  static constexpr size_t kBytes = (2 * static_cast<size_t>(kTcChunk) * kQS + kTcTile * kLS + kTcChunk * kLS) * 2 +
                                   (D + 8 * kTcChunk + 8) * 4;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads)
mlstm_outputs_kernel(const MlstmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int L = kTcChunk, TW = kTcTile, QS = OutputsLayout<D>::kQS, LS = OutputsLayout<D>::kLS;
  int e, chunk;
  if (!find_job(p, blockIdx.z, &e, &chunk)) return;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(raw);   // [L][QS]
  __nv_bfloat16* Ks = Qs + L * QS;                             // [L][QS]
  __nv_bfloat16* Vt = Ks + L * QS;                             // [TW][LS]
  __nv_bfloat16* Ws = Vt + TW * LS;                            // [L][LS]
  __nv_bfloat16* St = Ks;                                      // [TW][QS] in K's place, after the scores
  static_assert(kTcTile <= kTcChunk, "S^T must fit where K lay");
  float* ns = reinterpret_cast<float*>(Ws + L * LS);           // [D] n at the chunk's start
  float* av = ns + D;
  float* Mv = av + L;
  float* bv = Mv + L;
  float* lis = bv + L;
  float* lfs = lis + L;
  float* rs = lfs + L;       // [2][L]
  float* qn = rs + 2 * L;    // [L]
  const int d = D, dv = p.vdim;
  const bool wide = rows_wide(p);
  const int h = blockIdx.y, c0 = blockIdx.x * TW, job = blockIdx.z;
  const int cols = min(TW, dv - c0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int t0 = p.entry_starts[e], count = p.entry_starts[e + 1] - t0;
  const int start = chunk * L, len = min(L, count - start);
  const int rm = warp & 3, cn = warp >> 2;
  const float* rows = p.proj + static_cast<size_t>(t0 + start) * p.proj_width;
  const float m0 = p.chunk_aux[(static_cast<size_t>(job) * p.heads + h) * 4 + 2];
  const float* S_start = p.chunk_state + (static_cast<size_t>(job) * p.heads + h) * d * dv;
  const float* n_start = p.chunk_n + (static_cast<size_t>(job) * p.heads + h) * d;
  for (int dd = tid; dd < d; dd += kTcThreads) ns[dd] = n_start[dd];
  for (int item = tid; item < L * (D / 4); item += kTcThreads) {
    const int t = item / (D / 4), dd = (item % (D / 4)) * 4;
    float4 q = make_float4(0.0f, 0.0f, 0.0f, 0.0f), k = q;
    if (t < len) {
      const float* row = rows + static_cast<size_t>(t) * p.proj_width;
      q = load4(row + p.q_off + h * d + dd, wide);
      k = load4(row + p.k_off + h * d + dd, wide);
    }
    *reinterpret_cast<__nv_bfloat162*>(Qs + t * QS + dd) = __floats2bfloat162_rn(q.x * p.q_scale, q.y * p.q_scale);
    *reinterpret_cast<__nv_bfloat162*>(Qs + t * QS + dd + 2) = __floats2bfloat162_rn(q.z * p.q_scale, q.w * p.q_scale);
    *reinterpret_cast<__nv_bfloat162*>(Ks + t * QS + dd) = __floats2bfloat162_rn(k.x, k.y);
    *reinterpret_cast<__nv_bfloat162*>(Ks + t * QS + dd + 2) = __floats2bfloat162_rn(k.z, k.w);
  }
  for (int item = tid; item < L * TW; item += kTcThreads) {
    const int t = item / TW, c = item % TW;
    const float v = (t < len && c < cols) ? rows[static_cast<size_t>(t) * p.proj_width + p.v_off + h * dv + c0 + c] : 0.0f;
    Vt[c * LS + t] = __float2bfloat16_rn(v);
  }
  if (tid < L) {
    float li = 0.0f, lf = 0.0f;
    if (tid < len) {
      const float* row = rows + static_cast<size_t>(tid) * p.proj_width;
      li = capped(row[p.i_off + h], p.gate_cap);
      lf = log_sigmoid(capped(row[p.f_off + h], p.gate_cap));
    }
    lis[tid] = li;
    lfs[tid] = lf;
  }
  __syncthreads();
  if (warp == 0) {
    float first = lfs[2 * lane], second = lfs[2 * lane + 1];
    float pair = first + second, before = pair;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const float other = __shfl_up_sync(0xffffffffu, before, offset);
      if (lane >= offset) before += other;
    }
    const float b0 = before - pair + first, b1 = before;
    const float a0 = 2 * lane < len ? lis[2 * lane] - b0 : -INFINITY;
    const float a1 = 2 * lane + 1 < len ? lis[2 * lane + 1] - b1 : -INFINITY;
    // running maxima: M_t = max(m_0, a_0 .. a_t)
    float top = fmaxf(a0, a1), scan = top;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const float other = __shfl_up_sync(0xffffffffu, scan, offset);
      if (lane >= offset) scan = fmaxf(scan, other);
    }
    float earlier = __shfl_up_sync(0xffffffffu, scan, 1);
    if (lane == 0) earlier = -INFINITY;
    av[2 * lane] = a0;
    av[2 * lane + 1] = a1;
    bv[2 * lane] = b0;
    bv[2 * lane + 1] = b1;
    Mv[2 * lane] = fmaxf(m0, fmaxf(earlier, a0));
    Mv[2 * lane + 1] = fmaxf(m0, scan);
  }
  __syncthreads();
  {
    float G[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) G[j][i] = 0.0f;
#pragma unroll 4
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      load_a(a, Qs, QS, rm * 16, kk * 16, g, tq);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat16* at = Ks + (cn * 32 + j * 8 + g) * QS + kk * 16 + 2 * tq;
        mma_bf16(G[j], a, ld32(at), ld32(at + 8));
      }
    }
    float sums[2] = {0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int t = rm * 16 + g + 8 * r, s0 = cn * 32 + j * 8 + 2 * tq;
        float w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int sk = s0 + i;
          w[i] = (sk <= t && t < len) ? G[j][2 * r + i] * expf(av[sk] - Mv[t]) : 0.0f;
          sums[r] += w[i];
        }
        *reinterpret_cast<__nv_bfloat162*>(Ws + t * LS + s0) = __floats2bfloat162_rn(w[0], w[1]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sums[r] += __shfl_xor_sync(0xffffffffu, sums[r], 1);
      sums[r] += __shfl_xor_sync(0xffffffffu, sums[r], 2);
      if (tq == 0) rs[cn * L + rm * 16 + g + 8 * r] = sums[r];
    }
  }
  {
    const int t = tid >> 2, part = tid & 3;
    float sum = 0.0f;
    for (int dd = part; dd < D; dd += 4) sum = fmaf(__bfloat162float(Qs[t * QS + dd]), ns[dd], sum);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (part == 0) qn[t] = sum;
  }
  __syncthreads();
  // the state at the chunk's start, transposed, where K lay
  for (int item = tid; item < D * (TW / 4); item += kTcThreads) {
    const int dd = item / (TW / 4), c = (item % (TW / 4)) * 4;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (c + 3 < cols) v = *reinterpret_cast<const float4*>(S_start + static_cast<size_t>(dd) * dv + c0 + c);
    else {
      float* lanes = reinterpret_cast<float*>(&v);
      for (int i = 0; i < 4; ++i)
        if (c + i < cols) lanes[i] = S_start[static_cast<size_t>(dd) * dv + c0 + c + i];
    }
    St[c * QS + dd] = __float2bfloat16_rn(v.x);
    St[(c + 1) * QS + dd] = __float2bfloat16_rn(v.y);
    St[(c + 2) * QS + dd] = __float2bfloat16_rn(v.z);
    St[(c + 3) * QS + dd] = __float2bfloat16_rn(v.w);
  }
  __syncthreads();
  float O[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) O[j][i] = 0.0f;
#pragma unroll 4
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    load_a(a, Qs, QS, rm * 16, kk * 16, g, tq);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat16* at = St + (cn * 32 + j * 8 + g) * QS + kk * 16 + 2 * tq;
      mma_bf16(O[j], a, ld32(at), ld32(at + 8));
    }
  }
  float inter[2], denominator[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = rm * 16 + g + 8 * r;
    inter[r] = expf(m0 - Mv[t]);
    const float total = rs[t] + rs[L + t] + inter[r] * qn[t];
    denominator[r] = fmaxf(fabsf(total), expf(-(bv[t] + Mv[t]))) + p.denom_eps;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) O[j][i] *= inter[i >> 1];
#pragma unroll
  for (int kk = 0; kk < L / 16; ++kk) {
    uint32_t a[4];
    load_a(a, Ws, LS, rm * 16, kk * 16, g, tq);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat16* at = Vt + (cn * 32 + j * 8 + g) * LS + kk * 16 + 2 * tq;
      mma_bf16(O[j], a, ld32(at), ld32(at + 8));
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = rm * 16 + g + 8 * (i >> 1), c = cn * 32 + j * 8 + 2 * tq + (i & 1);
      if (t < len && c < cols)
        p.o_raw[(static_cast<size_t>(t0 + start + t) * p.heads + h) * dv + c0 + c] = O[j][i] / denominator[i >> 1];
    }
}

template <int D>
static int launch_chunks_at_once(const MlstmParams& p, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t error = cudaFuncSetAttribute(mlstm_parts_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(PartsLayout<D>::kBytes));
    if (error == cudaSuccess)
      error = cudaFuncSetAttribute(mlstm_outputs_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(OutputsLayout<D>::kBytes));
    if (error != cudaSuccess) return static_cast<int>(error);
    configured = true;
  }
  dim3 jobs((p.vdim + kTcTile - 1) / kTcTile, p.heads, p.max_jobs);
  int status = vipera_launch(mlstm_parts_kernel<D>, jobs, kTcThreads, PartsLayout<D>::kBytes, s, p);
  if (status != 0) return status;
  const size_t values = static_cast<size_t>(p.dim) * p.vdim;
  dim3 scan(static_cast<unsigned>((values / 4 + 255) / 256), p.heads, p.num_entries);
  status = vipera_launch(mlstm_scan_kernel, scan, 256, 0, s, p);
  if (status != 0) return status;
  return vipera_launch(mlstm_outputs_kernel<D>, jobs, kTcThreads, OutputsLayout<D>::kBytes, s, p);
}

template <int D>
static int launch_chunk_tc(const MlstmParams& p, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t error = cudaFuncSetAttribute(mlstm_chunk_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(TcLayout<D>::kBytes));
    if (error != cudaSuccess) return static_cast<int>(error);
    configured = true;
  }
  dim3 grid((p.vdim + kTcTile - 1) / kTcTile, p.heads, p.num_entries);
  return vipera_launch(mlstm_chunk_tc_kernel<D>, grid, kTcThreads, TcLayout<D>::kBytes, s, p);
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
// One block per (token, head).  out[t, h*dv + c] = o / rms(o) * weight[h*dv + c] * sigmoid(g[t, h*dv + c]).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_finish_kernel(const MlstmParams p, const float* __restrict__ weight, float eps, T* __restrict__ out,
                    const int* __restrict__ token_entry) {
  __shared__ float scratch_sum[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int dv = p.vdim, d = p.dim;
  const float* o = p.o_raw + (static_cast<size_t>(t) * p.heads + h) * dv;
  const float* gate = p.proj + static_cast<size_t>(t) * p.proj_width + p.g_off + h * dv;
  // up to four values a thread stay in registers between the two passes (value sizes up to 512)
  float mine[4], gates[4];
  float squares = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = tid + 128 * i;
    mine[i] = c < dv ? o[c] : 0.0f;
    gates[i] = c < dv ? gate[c] : 0.0f;
    squares = fmaf(mine[i], mine[i], squares);
  }
  for (int c = tid + 512; c < dv; c += 128) squares = fmaf(o[c], o[c], squares);
  squares = block_sum(squares, scratch_sum);
  const float inverse = rsqrtf(squares / static_cast<float>(dv) + eps);
  const float* w = weight + h * dv;
  T* dst = out + static_cast<size_t>(t) * p.heads * dv + h * dv;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = tid + 128 * i;
    if (c < dv) dst[c] = from_float<T>(mine[i] * inverse * w[c] * (1.0f / (1.0f + expf(-gates[i]))));
  }
  for (int c = tid + 512; c < dv; c += 128)
    dst[c] = from_float<T>(o[c] * inverse * w[c] * (1.0f / (1.0f + expf(-gate[c]))));
  const int e = token_entry[t];
  if (t == p.entry_starts[e + 1] - 1) {
    float* state = p.state + static_cast<long long>(p.state_slots[e]) * p.state_stride;
    float* n_state = state + static_cast<size_t>(p.heads) * d * dv + static_cast<size_t>(h) * d;
    float* m_state = state + static_cast<size_t>(p.heads) * d * (dv + 1) + h;
    const float* scratch = p.nm_scratch + (static_cast<size_t>(e) * p.heads + h) * (d + 1);
    for (int dd = tid; dd < d; dd += 128) n_state[dd] = scratch[dd];
    if (tid == 0) m_state[0] = scratch[d];
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

// Whether the tensor-core form of the chunk kernel takes these sizes.
VIPERA_API int vipera_mlstm_tc_takes(int dim) { return dim == 64 || dim == 128 || dim == 256; }

// Runs the cell over a step: `single` != 0 promises that every entry brings one token;
// `tensor_cores` != 0 allows the bfloat16 products of the tensor-core form for portions (a
// bfloat16 run; sizes it does not take run on the CUDA cores all the same).
// out is [tokens, heads * vdim] in `out_dtype`.
VIPERA_API int vipera_mlstm(const MlstmParams* params, int num_tokens, int single, int tensor_cores,
                            const float* norm_weight, float norm_eps, void* out, int out_dtype,
                            const int* token_entry, void* stream) {
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
  } else if (tensor_cores && vipera_mlstm_tc_takes(p.dim) && p.chunk_state && p.chunk_n && p.chunk_aux && p.max_jobs > 0 &&
             p.vdim % 4 == 0) {
    // all chunks at once (the caller gave the scratch for it: a long step)
    p.tile = kTcTile;
    status = p.dim == 64 ? launch_chunks_at_once<64>(p, s)
                         : p.dim == 128 ? launch_chunks_at_once<128>(p, s) : launch_chunks_at_once<256>(p, s);
  } else if (tensor_cores && vipera_mlstm_tc_takes(p.dim)) {
    p.tile = kTcTile;
    status = p.dim == 64 ? launch_chunk_tc<64>(p, s) : p.dim == 128 ? launch_chunk_tc<128>(p, s) : launch_chunk_tc<256>(p, s);
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
  dim3 grid(num_tokens, p.heads);
  if (out_dtype == VIPERA_F32)
    return vipera_launch(mlstm_finish_kernel<float>, grid, 128, 0, s, p, norm_weight, norm_eps, static_cast<float*>(out),
                         token_entry);
  if (out_dtype == VIPERA_BF16)
    return vipera_launch(mlstm_finish_kernel<__nv_bfloat16>, grid, 128, 0, s, p, norm_weight, norm_eps,
                         static_cast<__nv_bfloat16*>(out), token_entry);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API const char* vipera_mlstm_status_text(int status) { return vipera_status_text(status); }
