// Mixing over time channel by channel: what a sequence keeps is a vector, one number (or a few) per channel.
//
//   residual_conv   out_t = x_t + sum_j w[c, j] x_(t - taps + 1 + j)   a short causal convolution per channel, added to
//                   its own input; zeros before the sequence's start; the last taps - 1 inputs are the sequence's state
//   conv_keep       the last taps - 1 inputs of every sequence, kept for the next step
//   min_gru         S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, z = sigmoid(a), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
//                   out_t = S_t * silu(g_t).  a, u, g are the 32-bit sums of the projections; S is 32-bit and carried on.
//
// All arithmetic is 32-bit.  The recurrence is linear in S, so a sequence's rows of a step are cut into chunks that
// are walked side by side: each chunk first as a map S -> A S + B, then, from the state the chunks before it leave,
// once more for the outputs.  One row is one chunk: a plain update.
#include "common.cuh"

using namespace kvad;

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// A block per (row, chunk of 512 channels).  Inputs before the step's first row of the sequence come from the kept
// inputs [taps - 1, channels] (the oldest first), inputs before position 0 are zero.  `shift`: every sequence brings
// one row, so the thread that owns (row, channel) also moves the kept inputs on by one - no other block reads them.
template <typename T>
__global__ void __launch_bounds__(128)
residual_conv_kernel(const T* __restrict__ x, int64_t ld_x, const T* __restrict__ taps, T* __restrict__ out, int64_t ld_out,
                     float* __restrict__ state, int64_t state_stride, int64_t state_off, const int* __restrict__ row_seq,
                     const int* __restrict__ row_pos, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                     int channels, int n_taps, int shift) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, s = row_seq[r], pos = row_pos[r], first = seq_starts[s];
  const int p0 = pos - (r - first), keep = n_taps - 1;
  float* kept = state + (int64_t)seq_slots[s] * state_stride + state_off;
  const int lo = blockIdx.y * 512, hi = min(lo + 512, channels);
#pragma unroll 2
  for (int c = lo + threadIdx.x; c < hi; c += 128) {
    const float own = to_f32(x[(int64_t)r * ld_x + c]);
    float acc = 0.f, old[15];
    for (int j = 0; j < keep; ++j) {
      const int pp = pos - keep + j;
      float xv = 0.f;
      if (pp >= p0) xv = to_f32(x[(int64_t)(first + pp - p0) * ld_x + c]);
      else if (pp >= 0) xv = kept[(int64_t)(pp - p0 + keep) * channels + c];
      if (j < 15) old[j] = xv;
      acc = fmaf(to_f32(taps[(int64_t)c * n_taps + j]), xv, acc);
    }
    acc = fmaf(to_f32(taps[(int64_t)c * n_taps + keep]), own, acc);
    out[(int64_t)r * ld_out + c] = from_f32<T>(own + acc);
    if (shift) {
      for (int j = 0; j + 1 < keep; ++j) kept[(int64_t)j * channels + c] = old[j + 1];
      if (keep > 0) kept[(int64_t)(keep - 1) * channels + c] = own;
    }
  }
}

// Prompt rows in bfloat16 with up to four taps, channels in 16-byte pieces: a thread owns 8 channels of `rows_each`
// consecutive rows of the step.  The taps' weights and the window of the last taps - 1 inputs stay in registers; the
// window is read anew where a row opens another sequence (or the thread's run), so a row costs one 16-byte load and
// one store.  The sums run in the order of `residual_conv_kernel`: the same bits.
template <int NT>
__global__ void __launch_bounds__(64)
residual_conv_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x, const __nv_bfloat16* __restrict__ taps,
                          __nv_bfloat16* __restrict__ out, int64_t ld_out, const float* __restrict__ state, int64_t state_stride,
                          int64_t state_off, const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                          const int* __restrict__ seq_starts, const int* __restrict__ seq_slots, int n_rows, int channels, int rows_each) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KEEP = NT - 1;
  const int c = (blockIdx.y * 64 + threadIdx.x) * 8;
  if (c >= channels) return;
  float w[NT][8];
  {
    __nv_bfloat16 flat[8 * NT];                        // taps[c .. c + 8][0 .. NT): 16 NT bytes on a 16-byte boundary
#pragma unroll
    for (int v = 0; v < NT; ++v) *reinterpret_cast<uint4*>(flat + 8 * v) = *reinterpret_cast<const uint4*>(taps + (int64_t)c * NT + 8 * v);
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) w[j][i] = __bfloat162float(flat[i * NT + j]);
  }
  float win[KEEP > 0 ? KEEP : 1][8];
  const int r0 = blockIdx.x * rows_each, r1 = min(r0 + rows_each, n_rows);
  int s_before = -1;
  for (int r = r0; r < r1; ++r) {
    const int s = row_seq[r];
    __nv_bfloat16 in[8];
    *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(x + (int64_t)r * ld_x + c);
    if (KEEP > 0 && s != s_before) {
      const int pos = row_pos[r], first = seq_starts[s], p0 = pos - (r - first);
      const float* kept = state + (int64_t)seq_slots[s] * state_stride + state_off;
#pragma unroll
      for (int j = 0; j < KEEP; ++j) {
        const int pp = pos - KEEP + j;
        if (pp >= p0) {
          __nv_bfloat16 b[8];
          *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(x + (int64_t)(first + pp - p0) * ld_x + c);
#pragma unroll
          for (int i = 0; i < 8; ++i) win[j][i] = __bfloat162float(b[i]);
        } else if (pp >= 0) {
          const float4* k4 = reinterpret_cast<const float4*>(kept + (int64_t)(pp - p0 + KEEP) * channels + c);
          const float4 a = k4[0], b = k4[1];
          win[j][0] = a.x, win[j][1] = a.y, win[j][2] = a.z, win[j][3] = a.w;
          win[j][4] = b.x, win[j][5] = b.y, win[j][6] = b.z, win[j][7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) win[j][i] = 0.f;
        }
      }
      s_before = s;
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float own = __bfloat162float(in[i]);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < KEEP; ++j) acc = fmaf(w[j][i], win[j][i], acc);
      acc = fmaf(w[KEEP][i], own, acc);
      o[i] = from_f32<__nv_bfloat16>(own + acc);
#pragma unroll
      for (int j = 0; j + 1 < KEEP; ++j) win[j][i] = win[j + 1][i];
      if (KEEP > 0) win[KEEP - 1][i] = own;
    }
    *reinterpret_cast<uint4*>(out + (int64_t)r * ld_out + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// A thread per (sequence, channel): the inputs at the sequence's last taps - 1 positions, from this step's rows or,
// where the step brought fewer, from what was kept before.
template <typename T>
__global__ void conv_keep_kernel(const T* __restrict__ x, int64_t ld_x, float* __restrict__ state, int64_t state_stride,
                                 int64_t state_off, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                 int n_seqs, int channels, int n_taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n_seqs * channels) return;
  const int s = (int)(i / channels), c = (int)(i - (int64_t)s * channels);
  const int first = seq_starts[s], n_new = seq_starts[s + 1] - first, keep = n_taps - 1;
  float* kept = state + (int64_t)seq_slots[s] * state_stride + state_off;
  float old[15];
  for (int j = 0; j < keep; ++j) old[j] = kept[(int64_t)j * channels + c];
  for (int j = 0; j < keep; ++j) {
    const int from_new = n_new - keep + j;          // index among this step's rows, if not negative
    kept[(int64_t)j * channels + c] = from_new >= 0 ? to_f32(x[(int64_t)(first + from_new) * ld_x + c]) : old[j + n_new];
  }
}

constexpr int GRU_AHEAD = 8;            // rows whose sums a thread fetches before it walks them

__device__ __forceinline__ void gru_terms(float a, float u, float& z, float& cand) {
  z = sigmoid_f(a);
  cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
}

// Block (W channels, n_chunks chunks) per (W channels, sequence), W = blockDim.x: 32, or 16 where that leaves too few blocks.  zug: [rows, ld] with the three projections at
// columns off_z, off_u, off_g.
template <typename T>
__global__ void __launch_bounds__(1024)
min_gru_kernel(const float* __restrict__ zug, int64_t ld, int off_z, int off_u, int off_g, T* __restrict__ out, int64_t ld_out,
               float* __restrict__ state, int64_t state_stride, int64_t state_off, const int* __restrict__ seq_starts,
               const int* __restrict__ seq_slots, int width) {
  extern __shared__ float sm[];            // A [chunks][W], B [chunks][W]
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y, W = blockDim.x, c = blockIdx.x * W + threadIdx.x, j = threadIdx.y, n_chunks = blockDim.y;
  const int first = seq_starts[s], n_new = seq_starts[s + 1] - first;
  const int per = (n_new + n_chunks - 1) / n_chunks;
  const int lo = min(j * per, n_new), hi = min(lo + per, n_new);
  const bool live = c < width;
  float* A = sm;
  float* B = sm + n_chunks * W;
  if (n_chunks > 1) {
    float a_run = 1.f, b_run = 0.f;
    if (live) {
      for (int t0 = lo; t0 < hi; t0 += GRU_AHEAD) {          // the loads of GRU_AHEAD rows are in flight together
        float a[GRU_AHEAD], u[GRU_AHEAD];
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
          const float* row = zug + (int64_t)(first + min(t0 + i, hi - 1)) * ld;
          a[i] = row[off_z + c], u[i] = row[off_u + c];
        }
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
          if (t0 + i >= hi) break;
          float z, cand;
          gru_terms(a[i], u[i], z, cand);
          a_run *= 1.f - z;
          b_run = fmaf(z, cand, (1.f - z) * b_run);
        }
      }
    }
    A[j * W + threadIdx.x] = a_run;
    B[j * W + threadIdx.x] = b_run;
    __syncthreads();
  }
  if (!live) return;
  float* kept = state + (int64_t)seq_slots[s] * state_stride + state_off + c;
  float S = *kept;
  for (int i = 0; i < j; ++i) S = fmaf(A[i * W + threadIdx.x], S, B[i * W + threadIdx.x]);
  for (int t0 = lo; t0 < hi; t0 += GRU_AHEAD) {
    float a[GRU_AHEAD], u[GRU_AHEAD], g[GRU_AHEAD];
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      const float* row = zug + (int64_t)(first + min(t0 + i, hi - 1)) * ld;
      a[i] = row[off_z + c], u[i] = row[off_u + c], g[i] = row[off_g + c];
    }
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      if (t0 + i >= hi) break;
      float z, cand;
      gru_terms(a[i], u[i], z, cand);
      S = fmaf(z, cand, (1.f - z) * S);
      out[(int64_t)(first + t0 + i) * ld_out + c] = from_f32<T>(S * silu_f(g[i]));
    }
  }
  if (hi == n_new && (lo < hi || j == 0)) *kept = S;       // the chunk that holds the last row (an empty step: nothing changes)
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0, v = 0;
    n = (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) ? v : 148;
  }
  return n;
}

}  // namespace

KVAD_EXPORT int kvad_residual_conv(int dtype, const void* x, int64_t ld_x, const void* taps, void* out, int64_t ld_out, float* state,
                                   int64_t state_stride, int64_t state_off, const int* row_seq, const int* row_pos, const int* seq_starts,
                                   const int* seq_slots, int n_rows, int channels, int n_taps, int shift, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && channels > 0 && n_taps >= 1 && n_taps <= 16, "residual_conv: 1 to 16 taps, got %d", n_taps);
  KVAD_REQUIRE(x && taps && out && state && ld_x >= channels && ld_out >= channels, "residual_conv: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (dtype == KVAD_DTYPE_BF16 && !shift && n_taps <= 4 && n_rows >= 64 && channels % 8 == 0 && ld_x % 8 == 0 && ld_out % 8 == 0 &&
      state_stride % 4 == 0 && state_off % 4 == 0 && !misaligned(x) && !misaligned(out) && !misaligned(taps) && !misaligned(state)) {
    const int rows_each = 4;
    dim3 vgrid((n_rows + rows_each - 1) / rows_each, (channels + 511) / 512), vblock(64);
#define KVAD_CONV_ROWS(NT)                                                                                                          \
  kvad_launch(residual_conv_rows_kernel<NT>, vgrid, vblock, 0, stream, (const __nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)taps,    \
              (__nv_bfloat16*)out, ld_out, (const float*)state, state_stride, state_off, row_seq, row_pos, seq_starts, seq_slots,    \
              n_rows, channels, rows_each)
    if (n_taps == 1) KVAD_CONV_ROWS(1);
    else if (n_taps == 2) KVAD_CONV_ROWS(2);
    else if (n_taps == 3) KVAD_CONV_ROWS(3);
    else KVAD_CONV_ROWS(4);
#undef KVAD_CONV_ROWS
    KVAD_CHECK_LAUNCH("residual_conv");
    return KVAD_OK;
  }
  dim3 grid(n_rows, (channels + 511) / 512), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(residual_conv_kernel<float>, grid, block, 0, stream, (const float*)x, ld_x, (const float*)taps, (float*)out, ld_out, state,
                state_stride, state_off, row_seq, row_pos, seq_starts, seq_slots, channels, n_taps, shift);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(residual_conv_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)taps,
                (__nv_bfloat16*)out, ld_out, state, state_stride, state_off, row_seq, row_pos, seq_starts, seq_slots, channels, n_taps, shift);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "residual_conv: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("residual_conv");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_conv_keep(int dtype, const void* x, int64_t ld_x, float* state, int64_t state_stride, int64_t state_off,
                               const int* seq_starts, const int* seq_slots, int n_seqs, int channels, int n_taps, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && channels > 0 && n_taps >= 1 && n_taps <= 16, "conv_keep: bad sizes");
  if (n_seqs == 0 || n_taps == 1) return KVAD_OK;
  const int64_t total = (int64_t)n_seqs * channels;
  dim3 grid((unsigned)((total + 127) / 128)), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(conv_keep_kernel<float>, grid, block, 0, stream, (const float*)x, ld_x, state, state_stride, state_off, seq_starts, seq_slots,
                n_seqs, channels, n_taps);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(conv_keep_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ld_x, state, state_stride, state_off,
                seq_starts, seq_slots, n_seqs, channels, n_taps);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "conv_keep: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("conv_keep");
  return KVAD_OK;
}

// n_chunks: into how many chunks a sequence's rows of the step are cut (1..32; the caller chooses by the step's shape).
KVAD_EXPORT int kvad_min_gru(int out_dtype, const float* zug, int64_t ld, int off_z, int off_u, int off_g, void* out, int64_t ld_out,
                             float* state, int64_t state_stride, int64_t state_off, const int* seq_starts, const int* seq_slots,
                             int n_seqs, int width, int n_chunks, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && width > 0 && n_chunks >= 1 && n_chunks <= 32 && zug && out && state, "min_gru: bad arguments");
  KVAD_REQUIRE(ld >= width && ld_out >= width && state_stride >= state_off + width, "min_gru: rows or state shorter than the width");
  if (n_seqs == 0) return KVAD_OK;
  // 16 channels a block where 32 would leave SMs without one and the rows are walked in chunks (half a warp still reads whole sectors)
  const int per_block = (n_chunks > 1 && (int64_t)((width + 31) / 32) * n_seqs < sm_count()) ? 16 : 32;
  dim3 grid((width + per_block - 1) / per_block, n_seqs), block(per_block, n_chunks);
  const size_t smem = (size_t)2 * per_block * n_chunks * sizeof(float);
  if (out_dtype == KVAD_DTYPE_F32)
    kvad_launch(min_gru_kernel<float>, grid, block, smem, stream, zug, ld, off_z, off_u, off_g, (float*)out, ld_out, state, state_stride,
                state_off, seq_starts, seq_slots, width);
  else if (out_dtype == KVAD_DTYPE_BF16)
    kvad_launch(min_gru_kernel<__nv_bfloat16>, grid, block, smem, stream, zug, ld, off_z, off_u, off_g, (__nv_bfloat16*)out, ld_out, state,
                state_stride, state_off, seq_starts, seq_slots, width);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "min_gru: unknown dtype %d", out_dtype);
  KVAD_CHECK_LAUNCH("min_gru");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
