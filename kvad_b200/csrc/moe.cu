// A routed feed-forward: every row picks `top` of E experts, each a small gated feed-forward of its own.
//
//   moe_route        z = router logits (32-bit) -> the `top` largest (ties: the lower index), weights = softmax over
//                    the chosen logits only.  Mode 1 (scores): s = softmax(z) over all experts, the `top` largest of
//                    s + correction are chosen, weights = the chosen s over their sum (+ 1e-20)
//                    Experts from `n_real` on have no matrices (identity experts: their output is their input): their
//                    slots get no position (slot -> position = -1) and `moe_combine` adds weight * input for them
//   relu_squared     out = max(x, 0)^2, optionally times sigmoid(one number per row)
//   moe_sort         the (row, choice) slots grouped by expert, each expert's list padded to whole tiles of 32 (or 128)
//                    positions; tile -> expert, position -> row, position -> slot (-1: padding) and slot -> position
//   gather_rows      out[position] = a[row of the position] (zeros at padding): the operand of a product that reads
//                    whole tiles by TMA
//   grouped_linear   out[position] = W[expert of the position's tile] . a[row of the position]: a tiled product on
//                    the CUDA cores (32-bit sums in k order, so a row's bits do not depend on its tile's company),
//                    reading its rows and writing its outputs through the position lists
//   clamped_glu      g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(alpha g) (u + 1)
//   moe_combine      residual[row] += sum over the row's choices, in order, of weight * expert output (found through
//                    slot -> position)
//
// How many tiles a step can need depends only on its shape (rows x top / tile + E at most), so the launches do not
// depend on the routing and a step can be captured; tiles past the used ones leave at once.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int TM = 32, TN = 64, TK = 32;
constexpr int ROUTE_APART_ROWS = 256;      // from this many rows a step on, the routing is a launch of its own over many blocks

__device__ __forceinline__ void route_row_scores(const float* __restrict__ z, int n_experts, int top, const float* __restrict__ correction,
                                                 int* __restrict__ mine, float* __restrict__ wt) {
  float top_z = -INFINITY, total = 0.f;
  for (int e = 0; e < n_experts; ++e) top_z = fmaxf(top_z, z[e]);
  for (int e = 0; e < n_experts; ++e) total += expf(z[e] - top_z);
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.f;
    int at = -1;
    for (int e = 0; e < n_experts; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken = taken || mine[j] == e;
      const float sc = expf(z[e] - top_z) / total;
      const float v = sc + (correction ? correction[e] : 0.f);
      if (!taken && (at < 0 || v > best)) {
        best = v;
        best_s = sc;
        at = e;
      }
    }
    mine[k] = at;
    wt[k] = best_s;
    sum += best_s;
  }
  for (int k = 0; k < top; ++k) wt[k] /= sum + 1e-20f;
}

__device__ __forceinline__ void route_row(const float* __restrict__ logits, int64_t ld, int r, int n_experts, int top,
                                          int* __restrict__ chosen, float* __restrict__ weight, int mode = 0,
                                          const float* __restrict__ correction = nullptr) {
  const float* z = logits + (int64_t)r * ld;
  int* mine = chosen + (int64_t)r * top;
  float* wt = weight + (int64_t)r * top;
  if (mode == 1) {
    route_row_scores(z, n_experts, top, correction, mine, wt);
    return;
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = -1;
    for (int e = 0; e < n_experts; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken = taken || mine[j] == e;
      const float v = z[e];
      if (!taken && (at < 0 || v > best)) {
        best = v;
        at = e;
      }
    }
    mine[k] = at;
    wt[k] = best;
  }
  if (mode == 2) {      // every chosen expert weighs in with the sigmoid of its own logit (the same order: the sigmoid rises)
    for (int k = 0; k < top; ++k) wt[k] = 1.0f / (1.0f + expf(-wt[k]));
    return;
  }
  const float top_z = wt[0];
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    wt[k] = expf(wt[k] - top_z);
    sum += wt[k];
  }
  for (int k = 0; k < top; ++k) wt[k] /= sum;
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int64_t ld, int n_rows, int n_experts, int top,
                                 int* __restrict__ chosen, float* __restrict__ weight, int mode, const float* __restrict__ correction) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n_rows) route_row(logits, ld, r, n_experts, top, chosen, weight, mode, correction);
}

// One block.  counts -> padded offsets -> places.  Which place a slot gets inside its expert's list is not fixed
// (shared-memory atomics); no result depends on it.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(int* __restrict__ chosen, int n_slots, int top, int n_experts, int max_tiles, int tile_rows,
                int* __restrict__ tile_expert, int* __restrict__ pos_row, int* __restrict__ pos_slot, int* __restrict__ slot_pos,
                const float* __restrict__ logits, int64_t ld_logits, float* __restrict__ weight, int mode,
                const float* __restrict__ correction, int n_real) {
  extern __shared__ int sm[];
  int* counts = sm;
  int* offsets = sm + n_experts;
  int* cursor = sm + 2 * n_experts;
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = cursor[e] = 0;
  for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) pos_row[i] = pos_slot[i] = -1;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  if (logits != nullptr)                       // the routing itself first, a thread per row: one launch instead of two
    for (int r = threadIdx.x; r < n_slots / top; r += blockDim.x) route_row(logits, ld_logits, r, n_experts, top, chosen, weight, mode, correction);
  __syncthreads();
  for (int i = threadIdx.x; i < n_slots; i += blockDim.x)
    if (chosen[i] < n_real) atomicAdd(&counts[chosen[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < n_real; ++e) {
      offsets[e] = tile * tile_rows;
      const int n = (counts[e] + tile_rows - 1) / tile_rows;
      for (int t = 0; t < n; ++t) tile_expert[tile + t] = e;
      tile += n;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= n_real) {                  // an expert without matrices: nothing to multiply
      slot_pos[i] = -1;
      continue;
    }
    const int at = offsets[e] + atomicAdd(&cursor[e], 1);
    pos_row[at] = i / top;
    pos_slot[at] = i;
    slot_pos[i] = at;
  }
}

// A block per position; 16-byte pieces where `vec` says so.
template <typename T>
__global__ void __launch_bounds__(128)
gather_rows_kernel(const T* __restrict__ a, int64_t ld_a, const int* __restrict__ pos_row, T* __restrict__ out, int64_t ld_out, int width,
                   int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x, r = pos_row[p];
  T* o = out + (int64_t)p * ld_out;
  if (vec) {
    const int pieces = width * (int)sizeof(T) / 16;
    const uint4* src = r >= 0 ? reinterpret_cast<const uint4*>(a + (int64_t)r * ld_a) : nullptr;
    for (int i = threadIdx.x; i < pieces; i += 128) reinterpret_cast<uint4*>(o)[i] = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (int i = threadIdx.x; i < width; i += 128) o[i] = r >= 0 ? a[(int64_t)r * ld_a + i] : from_f32<T>(0.f);
  }
}

// Tile of 32 positions x 64 outputs, 256 threads, a thread 2 x 4 outputs; K in steps of 32 through shared memory, the next
// step's pieces on their way into registers while this one is multiplied (16-byte pieces where `vec` says the sizes and
// addresses allow).  A warp whose four positions are all padding stages its share and skips the arithmetic: with a few
// rows a step (decoding) most of a tile is padding and the kernel is a stream of the chosen experts' weights.
template <typename T, int N> struct Piece;
template <> struct Piece<float, 4> { using type = float4; };
template <> struct Piece<float, 8> { using type = float4; };
template <> struct Piece<__nv_bfloat16, 4> { using type = uint2; };
template <> struct Piece<__nv_bfloat16, 8> { using type = uint4; };

template <typename T, int N>
__device__ __forceinline__ void load_piece(const T* p, int n_left, bool vec, float* f) {
  if (vec && n_left >= N) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int j = 0; j < N; j += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + j);
        f[j] = v.x; f[j + 1] = v.y; f[j + 2] = v.z; f[j + 3] = v.w;
      }
    } else {
      const typename Piece<T, N>::type raw = *reinterpret_cast<const typename Piece<T, N>::type*>(p);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < N / 2; ++j) {
        const float2 v = __bfloat1622float2(h2[j]);
        f[2 * j] = v.x;
        f[2 * j + 1] = v.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = j < n_left ? to_f32(p[j]) : 0.f;
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const T* __restrict__ a, int64_t ld_a, const int* __restrict__ in_rows, const T* __restrict__ w,
                      int64_t expert_stride, TO* __restrict__ out, int64_t ld_out, const int* __restrict__ out_rows,
                      const int* __restrict__ valid, const int* __restrict__ tile_expert, int n_out, int k_dim, int vec) {
  __shared__ __align__(16) float As[TK][TM + 2];
  __shared__ __align__(16) float Ws[TK][TN + 4];
  __shared__ int rows_in[TM], rows_out[TM];
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y, expert = tile_expert[tile];
  if (expert < 0) return;
  const int n0 = blockIdx.x * TN, tid = threadIdx.x;
  if (tid < TM) {
    const int p = tile * TM + tid;
    const bool used = valid[p] >= 0;
    rows_in[tid] = used ? (in_rows ? in_rows[p] : p) : -1;
    rows_out[tid] = used ? (out_rows ? out_rows[p] : p) : -1;
  }
  __syncthreads();
  const T* we = w + (int64_t)expert * expert_stride;
  const int ty = tid >> 4, tx = tid & 15;
  const int warp_row = (tid >> 5) * 4;
  const bool busy = rows_out[warp_row] >= 0 || rows_out[warp_row + 1] >= 0 || rows_out[warp_row + 2] >= 0 || rows_out[warp_row + 3] >= 0;
  // staging shares: a thread carries 4 entries of one position's row and 8 entries of one output's weights
  const int am = tid >> 3, ak = (tid & 7) * 4, wn = tid >> 2, wk = (tid & 3) * 8;
  const int a_row = rows_in[am];
  const T* a_ptr = a_row >= 0 ? a + (int64_t)a_row * ld_a : nullptr;
  const T* w_ptr = n0 + wn < n_out ? we + (int64_t)(n0 + wn) * k_dim : nullptr;
  float ra[4], rw[8];
  auto fetch = [&](int k0) {
    if (a_ptr != nullptr) load_piece<T, 4>(a_ptr + k0 + ak, k_dim - k0 - ak, vec != 0, ra);
    else ra[0] = ra[1] = ra[2] = ra[3] = 0.f;
    if (w_ptr != nullptr) load_piece<T, 8>(w_ptr + k0 + wk, k_dim - k0 - wk, vec != 0, rw);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) rw[j] = 0.f;
    }
  };
  fetch(0);
  float acc[2][4] = {};
  for (int k0 = 0; k0 < k_dim; k0 += TK) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) As[ak + j][am] = ra[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) Ws[wk + j][wn] = rw[j];
    __syncthreads();
    if (k0 + TK < k_dim) fetch(k0 + TK);
    if (busy) {
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
        const float4 b = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
        acc[0][0] = fmaf(a0, b.x, acc[0][0]); acc[0][1] = fmaf(a0, b.y, acc[0][1]);
        acc[0][2] = fmaf(a0, b.z, acc[0][2]); acc[0][3] = fmaf(a0, b.w, acc[0][3]);
        acc[1][0] = fmaf(a1, b.x, acc[1][0]); acc[1][1] = fmaf(a1, b.y, acc[1][1]);
        acc[1][2] = fmaf(a1, b.z, acc[1][2]); acc[1][3] = fmaf(a1, b.w, acc[1][3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rows_out[ty * 2 + i];
    if (r < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < n_out) out[(int64_t)r * ld_out + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

// The same product for steps of a few rows (decoding): a stream of the chosen experts' weights.  A warp owns two outputs
// of one tile; its lanes take every 32nd 16-byte piece of the two weight rows (several on their way at once) and
// multiply them with the same pieces of up to eight of the tile's rows (which stay in the L1); a shuffle tree per
// (row, output) at the end.  A tile with more than eight rows streams its weights again per eight, from the L2.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
grouped_rows_kernel(const T* __restrict__ a, int64_t ld_a, const int* __restrict__ in_rows, const T* __restrict__ w,
                    int64_t expert_stride, TO* __restrict__ out, int64_t ld_out, const int* __restrict__ out_rows,
                    const int* __restrict__ valid, const int* __restrict__ tile_expert, int n_out, int k_dim) {
  constexpr int R = 8, CU = 2, PIECE = 16 / (int)sizeof(T);       // (four outputs a warp: 4 % slower on the step, fewer blocks and more registers)
  __shared__ int rows_in[TM], rows_out[TM], n_valid;
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y, expert = tile_expert[tile];
  if (expert < 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < TM) {                               // the tile's used positions, side by side
    const int p = tile * TM + tid;
    const bool used = valid[p] >= 0;
    const unsigned mask = __ballot_sync(0xffffffffu, used);
    if (used) {
      const int at = __popc(mask & ((1u << tid) - 1u));
      rows_in[at] = in_rows ? in_rows[p] : p;
      rows_out[at] = out_rows ? out_rows[p] : p;
    }
    if (tid == 0) n_valid = __popc(mask);
  }
  __syncthreads();
  const int col0 = (blockIdx.x * 8 + warp) * CU;
  if (col0 >= n_out) return;
  const T* we = w + (int64_t)expert * expert_stride;
  const T* wr[CU];
#pragma unroll
  for (int c = 0; c < CU; ++c) wr[c] = we + (int64_t)(col0 + c < n_out ? col0 + c : col0) * k_dim;
  for (int r0 = 0; r0 < n_valid; r0 += R) {
    const int nr = min(R, n_valid - r0);
    float acc[R][CU] = {};
#pragma unroll 4
    for (int k = lane * PIECE; k < k_dim; k += 32 * PIECE) {
      float wv[CU][PIECE], av[PIECE];
#pragma unroll
      for (int c = 0; c < CU; ++c) load_piece<T, PIECE>(wr[c] + k, PIECE, true, wv[c]);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r < nr) {
          load_piece<T, PIECE>(a + (int64_t)rows_in[r0 + r] * ld_a + k, PIECE, true, av);
#pragma unroll
          for (int j = 0; j < PIECE; ++j) {
#pragma unroll
            for (int c = 0; c < CU; ++c) acc[r][c] = fmaf(av[j], wv[c][j], acc[r][c]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r < nr) {
        float sums[CU];
#pragma unroll
        for (int c = 0; c < CU; ++c) sums[c] = warp_sum(acc[r][c]);
        if (lane == 0) {
          TO* o = out + (int64_t)rows_out[r0 + r] * ld_out + col0;
#pragma unroll
          for (int c = 0; c < CU; ++c)
            if (col0 + c < n_out) o[c] = from_f32<TO>(sums[c]);
        }
      }
    }
  }
}

__device__ __forceinline__ float clamped_glu_f(float gate, float up, float limit, float alpha) {
  const float g = fminf(gate, limit);
  const float u = fminf(fmaxf(up, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

// Eight neighbouring columns a thread, as 16-byte pieces (bfloat16 with sizes and addresses in whole pieces).
__global__ void clamped_glu_vec_kernel(const __nv_bfloat16* __restrict__ gate, int64_t ld_g, const __nv_bfloat16* __restrict__ up, int64_t ld_u,
                                       __nv_bfloat16* __restrict__ out, int64_t ld_o, int n_rows, int width, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 8;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = (int)(i - r * per_row) * 8;
    float g[8], u[8];
    load_piece<__nv_bfloat16, 8>(gate + r * ld_g + c, 8, true, g);
    load_piece<__nv_bfloat16, 8>(up + r * ld_u + c, 8, true, u);
    __nv_bfloat162 y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      y[j] = __floats2bfloat162_rn(clamped_glu_f(g[2 * j], u[2 * j], limit, alpha), clamped_glu_f(g[2 * j + 1], u[2 * j + 1], limit, alpha));
    *reinterpret_cast<uint4*>(out + r * ld_o + c) = *reinterpret_cast<const uint4*>(y);
  }
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gate, int64_t ld_g, const T* __restrict__ up, int64_t ld_u, T* __restrict__ out,
                                   int64_t ld_o, int n_rows, int width, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    out[r * ld_o + c] = from_f32<T>(clamped_glu_f(to_f32(gate[r * ld_g + c]), to_f32(up[r * ld_u + c]), limit, alpha));
  }
}

// out = act(s g) * (s u), s = scale[slot[p]] for position p (1 where `scale` is null or the position is padding):
// an expert that reads its input times the router's weight, W (s h) = s (W h), so the weight is applied to the two
// products' results instead of to their input.  act: 0 = silu, 3 = the tanh form of GELU.  32-bit arithmetic.
template <typename T>
__global__ void scaled_glu_kernel(const T* __restrict__ gate, int64_t ld_g, const T* __restrict__ up, int64_t ld_u, T* __restrict__ out,
                                  int64_t ld_o, const int* __restrict__ slot, const float* __restrict__ scale, int n_rows, int width, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    float s = 1.f;
    if (slot != nullptr) {
      const int at = slot[r];
      if (at < 0) {                       // (padding may hold anything)
        out[r * ld_o + c] = from_f32<T>(0.f);
        continue;
      }
      s = scale[at];
    }
    const float g = s * to_f32(gate[r * ld_g + c]), u = s * to_f32(up[r * ld_u + c]);
    out[r * ld_o + c] = from_f32<T>((act == 0 ? g / (1.0f + expf(-g)) : gelu_tanh(g)) * u);
  }
}

// The same, eight neighbouring bfloat16 columns a thread (widths and strides in eights, 16-byte aligned bases).
__global__ void scaled_glu_vec_kernel(const __nv_bfloat16* __restrict__ gate, int64_t ld_g, const __nv_bfloat16* __restrict__ up, int64_t ld_u,
                                      __nv_bfloat16* __restrict__ out, int64_t ld_o, const int* __restrict__ slot, const float* __restrict__ scale,
                                      int n_rows, int width, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 8;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = (int)(i - r * per_row) * 8;
    __nv_bfloat16 y[8];
    float s = 1.f;
    bool live = true;
    if (slot != nullptr) {
      const int at = slot[r];
      live = at >= 0;
      if (live) s = scale[at];
    }
    if (live) {
      __nv_bfloat16 g[8], u[8];
      *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(gate + r * ld_g + c);
      *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(up + r * ld_u + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float gv = s * __bfloat162float(g[e]), uv = s * __bfloat162float(u[e]);
        y[e] = __float2bfloat16_rn((act == 0 ? gv / (1.0f + expf(-gv)) : gelu_tanh(gv)) * uv);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = __float2bfloat16_rn(0.f);
    }
    *reinterpret_cast<uint4*>(out + r * ld_o + c) = *reinterpret_cast<const uint4*>(y);
  }
}

// out = max(x, 0)^2, times sigmoid(row_gate[r * ld_gate]) where a gate is given (one number per row).
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ x, int64_t ld_x, T* __restrict__ out, int64_t ld_o, const T* __restrict__ row_gate,
                                    int64_t ld_gate, int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    const float v = fmaxf(to_f32(x[r * ld_x + c]), 0.f);
    float y = v * v;
    if (row_gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(row_gate[r * ld_gate])));
    out[r * ld_o + c] = from_f32<T>(y);
  }
}

// The same, eight neighbouring bfloat16 columns a thread (widths and strides in eights, 16-byte aligned bases).
__global__ void relu_squared_vec_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x, __nv_bfloat16* __restrict__ out, int64_t ld_o,
                                        const __nv_bfloat16* __restrict__ row_gate, int64_t ld_gate, int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 8;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = (int)(i - r * per_row) * 8;
    __nv_bfloat16 v[8];
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(x + r * ld_x + c);
    const float g = row_gate != nullptr ? 1.0f / (1.0f + expf(-to_f32(row_gate[r * ld_gate]))) : 1.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float a = fmaxf(to_f32(v[k]), 0.f);
      float y = a * a;
      if (row_gate != nullptr) y *= g;
      v[k] = from_f32<__nv_bfloat16>(y);
    }
    *reinterpret_cast<uint4*>(out + r * ld_o + c) = *reinterpret_cast<const uint4*>(v);
  }
}

// Four neighbouring columns a thread (widths and strides in fours, 16-byte aligned bases); the choices in the same order.
template <typename T>
__global__ void moe_combine_vec_kernel(float* __restrict__ residual, const float* __restrict__ outs, int64_t ld_outs,
                                       const int* __restrict__ slot_pos, const float* __restrict__ weight, int n_rows, int width, int top,
                                       const T* __restrict__ input, int64_t ld_in) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 4;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = (int)(i - r * per_row) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top; ++k) {
      const float wk = weight ? weight[r * top + k] : 1.f;
      const int at = slot_pos[r * top + k];
      float4 v;
      if (at >= 0) v = *reinterpret_cast<const float4*>(outs + (int64_t)at * ld_outs + c);
      else v = make_float4(to_f32(input[r * ld_in + c]), to_f32(input[r * ld_in + c + 1]), to_f32(input[r * ld_in + c + 2]), to_f32(input[r * ld_in + c + 3]));
      acc.x = fmaf(wk, v.x, acc.x); acc.y = fmaf(wk, v.y, acc.y); acc.z = fmaf(wk, v.z, acc.z); acc.w = fmaf(wk, v.w, acc.w);
    }
    float4* at = reinterpret_cast<float4*>(residual + r * width + c);
    float4 x = *at;
    x.x += acc.x; x.y += acc.y; x.z += acc.z; x.w += acc.w;
    *at = x;
  }
}

template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ residual, const float* __restrict__ outs, int64_t ld_outs,
                                   const int* __restrict__ slot_pos, const float* __restrict__ weight, int n_rows, int width, int top,
                                   const T* __restrict__ input, int64_t ld_in) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int at = slot_pos[r * top + k];
      acc = fmaf(weight ? weight[r * top + k] : 1.f, at >= 0 ? outs[(int64_t)at * ld_outs + c] : to_f32(input[r * ld_in + c]), acc);
    }
    residual[i] += acc;
  }
}

inline int flat_blocks(int64_t total, int threads) {
  const int64_t b = (total + threads - 1) / threads;
  return (int)(b < 148 * 16 ? (b < 1 ? 1 : b) : 148 * 16);
}

}  // namespace

KVAD_EXPORT int kvad_moe_tile_rows() { return TM; }
KVAD_EXPORT int kvad_moe_route_apart_rows() { return ROUTE_APART_ROWS; }

KVAD_EXPORT int kvad_moe_route(const float* logits, int64_t ld, int n_rows, int n_experts, int top, int* chosen, float* weight,
                               cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_experts > 0 && top > 0 && top <= n_experts && ld >= n_experts, "moe_route: bad sizes experts=%d top=%d", n_experts, top);
  if (n_rows == 0) return KVAD_OK;
  kvad_launch(moe_route_kernel, dim3((n_rows + 63) / 64), dim3(64), 0, stream, logits, ld, n_rows, n_experts, top, chosen, weight, 0,
              (const float*)nullptr);
  KVAD_CHECK_LAUNCH("moe_route");
  return KVAD_OK;
}

// logits given: the rows are routed first (`chosen` and `weight` are written), then grouped.
KVAD_EXPORT int kvad_moe_sort(int* chosen, int n_slots, int top, int n_experts, int max_tiles, int tile_rows, int* tile_expert,
                              int* pos_row, int* pos_slot, int* slot_pos, const float* logits, int64_t ld_logits, float* weight,
                              int mode, const float* correction, int n_real, cudaStream_t stream) {
  KVAD_REQUIRE((mode == 0 || mode == 1 || mode == 2) && n_real >= 0 && n_real <= n_experts, "moe_sort: bad routing mode or expert counts");
  KVAD_REQUIRE(n_slots >= 0 && top > 0 && n_experts > 0 && n_experts <= 4096 && tile_rows > 0, "moe_sort: bad sizes");
  KVAD_REQUIRE(logits == nullptr || (weight != nullptr && top <= n_experts && ld_logits >= n_experts), "moe_sort: routing needs weights to write");
  KVAD_REQUIRE(max_tiles >= n_slots || max_tiles >= n_slots / tile_rows + n_real, "moe_sort: %d tiles cannot hold %d slots of %d experts",
               max_tiles, n_slots, n_experts);
  if (n_slots == 0) return KVAD_OK;
  if (logits != nullptr && n_slots / top >= ROUTE_APART_ROWS) {      // many rows: routed by many blocks first (by the step's shape only)
    const int n_rows = n_slots / top;
    kvad_launch(moe_route_kernel, dim3((n_rows + 63) / 64), dim3(64), 0, stream, logits, ld_logits, n_rows, n_experts, top, chosen, weight, mode,
                correction);
    KVAD_CHECK_LAUNCH("moe_route");
    logits = nullptr;
  }
  kvad_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * n_experts * sizeof(int), stream, chosen, n_slots, top, n_experts, max_tiles,
              tile_rows, tile_expert, pos_row, pos_slot, slot_pos, logits, ld_logits, weight, mode, correction, n_real);
  KVAD_CHECK_LAUNCH("moe_sort");
  return KVAD_OK;
}

// Position p reads row in_rows[p] of `a` (null: row p) and writes row out_rows[p] of `out` (null: row p); valid[p] < 0: padding.
// few_rows: the step has so few rows that most of a tile is padding; where the sizes allow 16-byte pieces the weight-streaming
// form runs.
KVAD_EXPORT int kvad_grouped_linear(int dtype, int out_f32, const void* a, int64_t ld_a, const int* in_rows, const void* w,
                                    int64_t expert_stride, void* out, int64_t ld_out, const int* out_rows, const int* valid,
                                    const int* tile_expert, int max_tiles, int n_out, int k_dim, int few_rows, cudaStream_t stream) {
  KVAD_REQUIRE(max_tiles >= 0 && n_out > 0 && k_dim > 0 && a && w && out && valid && tile_expert, "grouped_linear: bad arguments");
  if (max_tiles == 0) return KVAD_OK;
  dim3 grid((n_out + TN - 1) / TN, max_tiles), block(256);
  // 16-byte pieces: K and the rows' stride in whole pieces, the bases on 16-byte boundaries
  const int piece = dtype == KVAD_DTYPE_F32 ? 4 : 8;
  const int vec = (k_dim % piece == 0 && ld_a % piece == 0 && expert_stride % piece == 0 &&
                   ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) ? 1 : 0;
  if (few_rows && vec) {
    dim3 rgrid((n_out + 15) / 16, max_tiles);
#define KVAD_GR(T, TO)                                                                                                     \
  kvad_launch(grouped_rows_kernel<T, TO>, rgrid, block, 0, stream, (const T*)a, ld_a, in_rows, (const T*)w, expert_stride, (TO*)out, \
              ld_out, out_rows, valid, tile_expert, n_out, k_dim)
    if (dtype == KVAD_DTYPE_F32) KVAD_GR(float, float);
    else if (dtype == KVAD_DTYPE_BF16 && out_f32) KVAD_GR(__nv_bfloat16, float);
    else if (dtype == KVAD_DTYPE_BF16) KVAD_GR(__nv_bfloat16, __nv_bfloat16);
    else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "grouped_linear: unknown dtype %d", dtype);
#undef KVAD_GR
    KVAD_CHECK_LAUNCH("grouped_linear");
    return KVAD_OK;
  }
#define KVAD_GL(T, TO)                                                                                                       \
  kvad_launch(grouped_linear_kernel<T, TO>, grid, block, 0, stream, (const T*)a, ld_a, in_rows, (const T*)w, expert_stride, (TO*)out, \
              ld_out, out_rows, valid, tile_expert, n_out, k_dim, vec)
  if (dtype == KVAD_DTYPE_F32) KVAD_GL(float, float);
  else if (dtype == KVAD_DTYPE_BF16 && out_f32) KVAD_GL(__nv_bfloat16, float);
  else if (dtype == KVAD_DTYPE_BF16) KVAD_GL(__nv_bfloat16, __nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "grouped_linear: unknown dtype %d", dtype);
#undef KVAD_GL
  KVAD_CHECK_LAUNCH("grouped_linear");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_clamped_glu(int dtype, const void* gate, int64_t ld_g, const void* up, int64_t ld_u, void* out, int64_t ld_o,
                                 int n_rows, int width, float limit, float alpha, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && limit > 0.f, "clamped_glu: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(clamped_glu_kernel<float>, grid, block, 0, stream, (const float*)gate, ld_g, (const float*)up, ld_u, (float*)out, ld_o, n_rows,
                width, limit, alpha);
  else if (dtype == KVAD_DTYPE_BF16 && width % 8 == 0 && ld_g % 8 == 0 && ld_u % 8 == 0 && ld_o % 8 == 0 &&
           ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
    kvad_launch(clamped_glu_vec_kernel, dim3(flat_blocks((int64_t)n_rows * (width / 8), 256)), block, 0, stream, (const __nv_bfloat16*)gate, ld_g,
                (const __nv_bfloat16*)up, ld_u, (__nv_bfloat16*)out, ld_o, n_rows, width, limit, alpha);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(clamped_glu_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)gate, ld_g, (const __nv_bfloat16*)up, ld_u,
                (__nv_bfloat16*)out, ld_o, n_rows, width, limit, alpha);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "clamped_glu: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("clamped_glu");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_gather_rows(int dtype, const void* a, int64_t ld_a, const int* pos_row, void* out, int64_t ld_out, int n_pos, int width,
                                 cudaStream_t stream) {
  KVAD_REQUIRE(n_pos >= 0 && width > 0 && a && pos_row && out, "gather_rows: bad arguments");
  if (n_pos == 0) return KVAD_OK;
  const int es = dtype == KVAD_DTYPE_F32 ? 4 : 2;
  const int vec = ((width * es) % 16 == 0 && (ld_a * es) % 16 == 0 && (ld_out * es) % 16 == 0 &&
                   ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) ? 1 : 0;
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(gather_rows_kernel<float>, dim3(n_pos), dim3(128), 0, stream, (const float*)a, ld_a, pos_row, (float*)out, ld_out, width, vec);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(gather_rows_kernel<__nv_bfloat16>, dim3(n_pos), dim3(128), 0, stream, (const __nv_bfloat16*)a, ld_a, pos_row,
                (__nv_bfloat16*)out, ld_out, width, vec);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "gather_rows: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("gather_rows");
  return KVAD_OK;
}

// input (of `in_dtype`, may be null where every slot has a position): the rows the experts read, for slots without a position.
KVAD_EXPORT int kvad_moe_combine(float* residual, const float* outs, int64_t ld_outs, const int* slot_pos, const float* weight, int n_rows,
                                 int width, int top, int in_dtype, const void* input, int64_t ld_in, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && top > 0 && residual && outs && slot_pos, "moe_combine: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const bool vec = width % 4 == 0 && ld_outs % 4 == 0 && ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(outs)) & 15) == 0;
  dim3 grid(vec ? flat_blocks((int64_t)n_rows * (width / 4), 256) : flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (in_dtype == KVAD_DTYPE_BF16) {
    if (vec) kvad_launch(moe_combine_vec_kernel<__nv_bfloat16>, grid, block, 0, stream, residual, outs, ld_outs, slot_pos, weight, n_rows, width, top,
                         (const __nv_bfloat16*)input, ld_in);
    else kvad_launch(moe_combine_kernel<__nv_bfloat16>, grid, block, 0, stream, residual, outs, ld_outs, slot_pos, weight, n_rows, width, top,
                     (const __nv_bfloat16*)input, ld_in);
  } else {
    if (vec) kvad_launch(moe_combine_vec_kernel<float>, grid, block, 0, stream, residual, outs, ld_outs, slot_pos, weight, n_rows, width, top,
                         (const float*)input, ld_in);
    else kvad_launch(moe_combine_kernel<float>, grid, block, 0, stream, residual, outs, ld_outs, slot_pos, weight, n_rows, width, top,
                     (const float*)input, ld_in);
  }
  KVAD_CHECK_LAUNCH("moe_combine");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_relu_squared(int dtype, const void* x, int64_t ld_x, void* out, int64_t ld_o, const void* row_gate, int64_t ld_gate,
                                  int n_rows, int width, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && x && out, "relu_squared: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  if (dtype == KVAD_DTYPE_BF16 && width % 8 == 0 && ld_x % 8 == 0 && ld_o % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    kvad_launch(relu_squared_vec_kernel, dim3(flat_blocks((int64_t)n_rows * (width / 8), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)x,
                ld_x, (__nv_bfloat16*)out, ld_o, (const __nv_bfloat16*)row_gate, ld_gate, n_rows, width);
    KVAD_CHECK_LAUNCH("relu_squared");
    return KVAD_OK;
  }
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(relu_squared_kernel<float>, grid, block, 0, stream, (const float*)x, ld_x, (float*)out, ld_o, (const float*)row_gate, ld_gate, n_rows, width);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(relu_squared_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ld_x, (__nv_bfloat16*)out, ld_o,
                (const __nv_bfloat16*)row_gate, ld_gate, n_rows, width);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "relu_squared: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("relu_squared");
  return KVAD_OK;
}

// slot: for every row of gate / up the (row, choice) pair it stands for (-1: padding, whose output is zero), scale: one
// float32 per pair; both null: no scaling.
KVAD_EXPORT int kvad_scaled_glu(int dtype, const void* gate, int64_t ld_g, const void* up, int64_t ld_u, void* out, int64_t ld_o, const int* slot,
                                const float* scale, int n_rows, int width, int act, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && gate && up && out && (act == 0 || act == 3) && ((slot == nullptr) == (scale == nullptr)),
               "scaled_glu: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(scaled_glu_kernel<float>, grid, block, 0, stream, (const float*)gate, ld_g, (const float*)up, ld_u, (float*)out, ld_o, slot, scale,
                n_rows, width, act);
  else if (dtype == KVAD_DTYPE_BF16 && width % 8 == 0 && ld_g % 8 == 0 && ld_u % 8 == 0 && ld_o % 8 == 0 &&
           ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
    kvad_launch(scaled_glu_vec_kernel, dim3(flat_blocks((int64_t)n_rows * (width / 8), 256)), block, 0, stream, (const __nv_bfloat16*)gate, ld_g,
                (const __nv_bfloat16*)up, ld_u, (__nv_bfloat16*)out, ld_o, slot, scale, n_rows, width, act);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(scaled_glu_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)gate, ld_g, (const __nv_bfloat16*)up, ld_u,
                (__nv_bfloat16*)out, ld_o, slot, scale, n_rows, width, act);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "scaled_glu: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("scaled_glu");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
