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
// gla_scan_kernel: a block owns (a tile of 32 value columns, head, entry); warp r of the block
// holds rows r*ROWS .. r*ROWS+ROWS-1 of the tile's columns in registers (a lane a column) and
// walks the entry's tokens in order.  Each warp writes its share of o to a scratch
// [row shares][tokens][heads*dv]; gla_finish_kernel adds the shares in a fixed order and applies
// norm, gate and scale (a warp per (token, head)).
#include "common.cuh"

constexpr int kGlaMaxShares = 16;

struct GlaParams {
  const float* proj;      // [tokens, proj_width]: q, k, v, g at their offsets
  long long proj_width;
  int q_off, k_off, v_off, g_off;
  const float* z;         // [tokens, heads * dim]  decay pre-activations (bias included)
  float* state;           // [slots, heads * dim * vdim]
  const int* entry_starts;
  const int* state_slots;
  const int* fresh;
  float* partial;         // [shares][tokens][heads * vdim]
  const float* norm_weight;  // [vdim]
  void* out;              // [tokens, heads * vdim]
  int heads, dim, vdim, num_entries, num_tokens, shares;
  float q_scale, inv_tau, eps, out_scale;
};

template <int ROWS>
__global__ void __launch_bounds__(kGlaMaxShares * 32) gla_scan_kernel(const GlaParams p) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, share = threadIdx.x >> 5;
  const int column = blockIdx.x * 32 + lane;
  const int head = blockIdx.y, entry = blockIdx.z;
  const bool live = column < p.vdim;
  const int row0 = share * ROWS;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) s[r] = 0.0f;
  pdl_wait();
  const int first = p.entry_starts[entry], last = p.entry_starts[entry + 1];
  if (last <= first) return;
  float* state = p.state + (static_cast<size_t>(p.state_slots[entry]) * p.heads + head) * p.dim * p.vdim;
  if (live && !p.fresh[entry]) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < p.dim) s[r] = state[static_cast<size_t>(row0 + r) * p.vdim + column];
  }
  const size_t out_width = static_cast<size_t>(p.heads) * p.vdim;
  float* partial = p.partial + static_cast<size_t>(share) * p.num_tokens * out_width + head * p.vdim;
  for (int t = first; t < last; ++t) {
    const float* row = p.proj + static_cast<size_t>(t) * p.proj_width;
    const float* q = row + p.q_off + head * p.dim + row0;
    const float* k = row + p.k_off + head * p.dim + row0;
    const float* z = p.z + (static_cast<size_t>(t) * p.heads + head) * p.dim + row0;
    const float v = live ? row[p.v_off + head * p.vdim + column] : 0.0f;
    float o = 0.0f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (row0 + r < p.dim) {
        // log sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
        const float zz = z[r];
        const float alpha = expf((fminf(zz, 0.0f) - log1pf(expf(-fabsf(zz)))) * p.inv_tau);
        s[r] = fmaf(alpha, s[r], k[r] * v);
        o = fmaf(s[r], q[r] * p.q_scale, o);
      }
    }
    if (live) partial[static_cast<size_t>(t) * out_width + column] = o;
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < p.dim) state[static_cast<size_t>(row0 + r) * p.vdim + column] = s[r];
  }
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
  if (!p.proj || !p.z || !p.state || !p.entry_starts || !p.state_slots || !p.fresh || !p.partial || !p.norm_weight || !p.out)
    return VIPERA_BAD_ARGUMENT;
  const int rows = gla_rows(p.dim);
  p.shares = (p.dim + rows - 1) / rows;
  if (p.shares > kGlaMaxShares) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((p.vdim + 31) / 32, p.heads, p.num_entries);
  int status;
  if (rows == 8) status = vipera_launch(gla_scan_kernel<8>, grid, p.shares * 32, 0, s, p);
  else if (rows == 16) status = vipera_launch(gla_scan_kernel<16>, grid, p.shares * 32, 0, s, p);
  else status = vipera_launch(gla_scan_kernel<32>, grid, p.shares * 32, 0, s, p);
  if (status) return status;
  const int items = p.num_tokens * p.heads;
  if (out_dtype == VIPERA_BF16) return vipera_launch(gla_finish_kernel<__nv_bfloat16>, (items + 3) / 4, 128, 0, s, p);
  if (out_dtype == VIPERA_F32) return vipera_launch(gla_finish_kernel<float>, (items + 3) / 4, 128, 0, s, p);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_gla_params_size() { return static_cast<int>(sizeof(GlaParams)); }
