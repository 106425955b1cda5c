// Row-wise kernels of designs with RMS norms, rotary positions and gated activations.
// All arithmetic is 32-bit (sums of squares, angles, sines, gates); the element type only says how
// tensors are stored.
//
//   rmsnorm           y = x / sqrt(mean(x^2) + eps) * w      (w absent: 1; `unit_offset`: 1 + w)
//   residual_rmsnorm  x += mult * delta; delta = 0; y = rmsnorm(x)   - a block whose sublayers add into `delta`
//                     leaves the scaled sum to the next reader of the stream
//   rotary            pairs of a head's first `dims` entries turned by position * base^(-2i/dims), either
//                     entry i with i + dims/2 ("half") or 2i with 2i + 1 ("interleaved")
//                     (`inverse`: by the negative angle; `head_gate`: each head's turned entries times the sigmoid
//                     of one number per row and head)
//   gate_mul          out = act(a) * b,  act = silu, sigmoid, relu or the tanh form of GELU
//   scale_add         x += mult * delta; delta = 0
//   postnorm_rmsnorm  x += g * delta / rms(delta); delta = 0; y = rmsnorm(x)   - a block that norms a sublayer's result
//                     before it scales it into the stream leaves that to the next reader of the stream (y may be absent)
//   head_gate         x[r, h, :] *= sigmoid(gate[r, h])
//   stream_concat     out = [x | x0] in the compute dtype: two 32-bit streams side by side as one product's input
//   cast_rows         y = x in the compute dtype: what a sublayer that reads the stream itself multiplies with
//                     (postnorm_rmsnorm with a negative eps leaves the same beside the sum it takes up)
//   pair_norm_sum     delta += mult * (ga * a / rms(a) + gb * b / rms(b)); a = 0; b = 0   - two mixers side by side,
//                     each normed over the model width before they are averaged
//   tanh_cap          x = cap * tanh(x / cap) in place (32-bit logits)
#include "common.cuh"

using namespace kvad;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// A block of 128 threads per row.  Two passes over the row (the second finds it in the L1), four entries a thread
// and trip where the row allows 16-byte loads of 32-bit values: few trips, their loads in flight together.  The
// sums run thread by thread in column order, then a shuffle tree and the warps in order - a row's bits do not
// depend on its company.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
rmsnorm_kernel(const TI* __restrict__ x, int64_t ld_in, const int* __restrict__ row_index, const void* __restrict__ w,
               int w_f32, int unit_offset, TO* __restrict__ out, int64_t ld_out, int n_rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const TI* xr = x + (int64_t)(row_index ? row_index[r] : r) * ld_in;
  float sq = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float v = to_f32(xr[c]);
    sq = fmaf(v, v, sq);
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
  TO* o = out + (int64_t)r * ld_out;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    float g = 1.f;
    if (w != nullptr) g = load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f);
    o[c] = from_f32<TO>(to_f32(xr[c]) * inv * g);
  }
}

// The same on the 32-bit residual stream with a pending scaled sum: v = x + mult * delta.  With `write_back`
// (all rows are walked) v replaces x and delta is cleared for the sublayers of the next block; with a row
// list (the head reads a few rows) nothing is written back.  `vec`: the width is a multiple of 4 and the rows
// start on 16-byte boundaries.
template <typename TO>
__global__ void __launch_bounds__(128)
residual_rmsnorm_kernel(float* __restrict__ x, float* __restrict__ delta, float mult, int write_back,
                        const int* __restrict__ row_index, const void* __restrict__ w, int w_f32, int unit_offset,
                        TO* __restrict__ out, int64_t ld_out, int n_rows, int width, float eps, int vec) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int64_t src = (int64_t)(row_index ? row_index[r] : r) * width;
  float* xr = x + src;
  float* dr = delta + src;
  float sq = 0.f;
  if (vec) {
#pragma unroll 2
    for (int c = threadIdx.x * 4; c < width; c += 512) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + c), dv = *reinterpret_cast<const float4*>(dr + c);
      const float4 v = make_float4(fmaf(mult, dv.x, xv.x), fmaf(mult, dv.y, xv.y), fmaf(mult, dv.z, xv.z), fmaf(mult, dv.w, xv.w));
      if (write_back) {
        *reinterpret_cast<float4*>(xr + c) = v;
        *reinterpret_cast<float4*>(dr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += 128) {
      const float v = fmaf(mult, dr[c], xr[c]);
      if (write_back) {
        xr[c] = v;
        dr[c] = 0.f;
      }
      sq = fmaf(v, v, sq);
    }
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
  TO* o = out + (int64_t)r * ld_out;
  const int step = vec ? 4 : 1;
  for (int c0 = threadIdx.x * step; c0 < width; c0 += 128 * step) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = c0 + e;
      if (e < step) {
        const float v = write_back ? xr[c] : fmaf(mult, dr[c], xr[c]);     // (the thread reads what it wrote)
        float g = 1.f;
        if (w != nullptr) g = load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f);
        o[c] = from_f32<TO>(v * inv * g);
      }
    }
  }
}

__global__ void scale_add_kernel(float* __restrict__ x, float* __restrict__ delta, float mult, int64_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    x[i] = fmaf(mult, delta[i], x[i]);
    delta[i] = 0.f;
  }
}

// One thread per (row, head, pair).  `src` and `dst` may be the same buffer (each pair is read, then written, by
// one thread) or different ones (a copy that rotates).
template <typename T>
__global__ void rotary_kernel(const T* __restrict__ src, int64_t ld_src, int head_stride_src, int off_src,
                              T* __restrict__ dst, int64_t ld_dst, int head_stride_dst, int off_dst,
                              const int* __restrict__ row_pos, const float* __restrict__ inv_freq, int n_rows, int n_heads,
                              int dims, int interleaved, int inverse, const T* __restrict__ head_gate, int64_t ld_gate) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = dims / 2;
  const int64_t total = (int64_t)n_rows * n_heads * half;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int p = (int)(i % half), h = (int)((i / half) % n_heads), r = (int)(i / ((int64_t)half * n_heads));
    const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
    const T* s = src + (int64_t)r * ld_src + (int64_t)h * head_stride_src + off_src;
    T* d = dst + (int64_t)r * ld_dst + (int64_t)h * head_stride_dst + off_dst;
    float sn, cs;
    sincosf((float)row_pos[r] * inv_freq[p], &sn, &cs);
    if (inverse) sn = -sn;
    float g = 1.f;
    if (head_gate != nullptr) g = sigmoid_f(to_f32(head_gate[(int64_t)r * ld_gate + h]));
    const float u = to_f32(s[a]), v = to_f32(s[b]);
    d[a] = from_f32<T>(turn_first(u, v, cs, sn) * g);
    d[b] = from_f32<T>(turn_second(u, v, cs, sn) * g);
  }
}

template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, int64_t ld_a, const T* __restrict__ b, int64_t ld_b,
                                T* __restrict__ out, int64_t ld_out, int n_rows, int width, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    const float g = to_f32(a[(int64_t)r * ld_a + c]);
    const float v = to_f32(b[(int64_t)r * ld_b + c]);
    out[(int64_t)r * ld_out + c] = from_f32<T>((act == 0 ? silu_f(g) : act == 1 ? sigmoid_f(g) : act == 2 ? fmaxf(g, 0.f) : gelu_tanh(g)) * v);
  }
}

// x += g * delta / rms(delta) on the 32-bit stream (g: one 32-bit number per column), then y = rmsnorm(x) with `w`
// (y absent: only the sum).  With `write_back` (all rows are walked) the sum replaces x and delta is cleared; with a
// row list nothing is written back.  Two sums of squares per row, each in column order through the same tree.
// A negative `eps`: y = x as it is (no norm, no weight) - for a reader that wants the stream itself in its own dtype.
// IN_REGISTERS (few rows, up to 2048 columns): a row lies in its block's registers and every load is in flight before
// the first sum; the sums run in the same order, so both forms give the same bits.
template <typename TO, bool IN_REGISTERS>
__global__ void __launch_bounds__(128)
postnorm_rmsnorm_kernel(float* __restrict__ x, float* __restrict__ delta, const float* __restrict__ g, float eps_post, int write_back,
                        const int* __restrict__ row_index, const void* __restrict__ w, int w_f32, int unit_offset,
                        TO* __restrict__ out, int64_t ld_out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int64_t src = (int64_t)(row_index ? row_index[r] : r) * width;
  float* xr = x + src;
  float* dr = delta + src;
  constexpr int PER = 16;
  if (IN_REGISTERS) {
    float d[PER], xv[PER], gg[PER], ww[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int c = threadIdx.x + 128 * k;
      const bool in = c < width;
      d[k] = in ? dr[c] : 0.f;
      xv[k] = in ? xr[c] : 0.f;
      gg[k] = in ? g[c] : 0.f;
      ww[k] = (in && out != nullptr && w != nullptr) ? load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f) : 1.f;
    }
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k)
      if (threadIdx.x + 128 * k < width) sq = fmaf(d[k], d[k], sq);
    sq = block_sum(sq, scratch);
    const float inv_d = 1.0f / sqrtf(sq / (float)width + eps_post);
    float sq_x = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int c = threadIdx.x + 128 * k;
      if (c < width) {
        const float v = fmaf(d[k] * inv_d, gg[k], xv[k]);
        if (write_back) {
          xr[c] = v;
          dr[c] = 0.f;
        }
        sq_x = fmaf(v, v, sq_x);
        xv[k] = v;
      }
    }
    if (out == nullptr) return;
    sq_x = block_sum(sq_x, scratch);
    const float inv = eps < 0.f ? 1.f : 1.0f / sqrtf(sq_x / (float)width + eps);
    TO* o = out + (int64_t)r * ld_out;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int c = threadIdx.x + 128 * k;
      if (c < width) o[c] = from_f32<TO>(xv[k] * inv * ww[k]);
    }
    return;
  }
  float sq = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float v = dr[c];
    sq = fmaf(v, v, sq);
  }
  sq = block_sum(sq, scratch);
  const float inv_d = 1.0f / sqrtf(sq / (float)width + eps_post);
  float sq_x = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float v = fmaf(dr[c] * inv_d, g[c], xr[c]);
    if (write_back) {
      xr[c] = v;
      dr[c] = 0.f;
    }
    sq_x = fmaf(v, v, sq_x);
  }
  if (out == nullptr) return;
  sq_x = block_sum(sq_x, scratch);
  const float inv = eps < 0.f ? 1.f : 1.0f / sqrtf(sq_x / (float)width + eps);
  TO* o = out + (int64_t)r * ld_out;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float v = write_back ? xr[c] : fmaf(dr[c] * inv_d, g[c], xr[c]);      // (the thread reads what it wrote)
    float gain = 1.f;
    if (w != nullptr) gain = load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f);
    o[c] = from_f32<TO>(v * inv * gain);
  }
}

// y = x in the compute dtype (rows of the 32-bit stream, all of them or those a list names).
template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, const int* __restrict__ row_index, TO* __restrict__ out, int64_t ld_out,
                                 int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    out[r * ld_out + c] = from_f32<TO>(x[(int64_t)(row_index ? row_index[r] : r) * width + c]);
  }
}

// The same for widths and strides in fours: a thread takes four neighbouring columns (one 16-byte load).
template <typename TO>
__global__ void cast_rows_vec_kernel(const float* __restrict__ x, const int* __restrict__ row_index, TO* __restrict__ out, int64_t ld_out,
                                     int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 4;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = (int)(i - r * per_row) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + (int64_t)(row_index ? row_index[r] : r) * width + c);
    TO* o = out + r * ld_out + c;
    o[0] = from_f32<TO>(v.x); o[1] = from_f32<TO>(v.y); o[2] = from_f32<TO>(v.z); o[3] = from_f32<TO>(v.w);
  }
}

// delta += mult * (ga * a / rms(a) + gb * b / rms(b)); a = 0; b = 0 (all 32-bit, rows of `width`; ga, gb one number per
// column).  A block per row; the two sums of squares run in column order through the same tree.
__global__ void __launch_bounds__(128)
pair_norm_sum_kernel(float* __restrict__ a, float* __restrict__ b, const float* __restrict__ ga, const float* __restrict__ gb,
                     float* __restrict__ delta, int width, float eps, float mult) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  float* ar = a + (int64_t)blockIdx.x * width;
  float* br = b + (int64_t)blockIdx.x * width;
  float* dr = delta + (int64_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float u = ar[c], v = br[c];
    sa = fmaf(u, u, sa);
    sb = fmaf(v, v, sb);
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ia = 1.0f / sqrtf(sa / (float)width + eps), ib = 1.0f / sqrtf(sb / (float)width + eps);
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float u = ar[c] * ia * ga[c], v = br[c] * ib * gb[c];
    dr[c] = fmaf(mult, u + v, dr[c]);
    ar[c] = 0.f;
    br[c] = 0.f;
  }
}

__global__ void tanh_cap_kernel(float* __restrict__ x, int64_t total, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

// x[r, h * dv + d] *= sigmoid(gate[r, h]): one number per row and head.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, int64_t ld_x, const T* __restrict__ gate, int64_t ld_gate, int n_rows, int n_heads, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int width = n_heads * dv;
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width;
    const int c = (int)(i - r * width);
    T* at = x + r * ld_x + c;
    *at = from_f32<T>(to_f32(*at) * sigmoid_f(to_f32(gate[r * ld_gate + c / dv])));
  }
}

template <typename T>
__global__ void stream_concat_kernel(const float* __restrict__ x, const float* __restrict__ x0, T* __restrict__ out, int n_rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i - r * width;
    out[r * 2 * width + c] = from_f32<T>(x[i]);
    out[r * 2 * width + width + c] = from_f32<T>(x0[i]);
  }
}

inline int flat_blocks(int64_t total, int threads) {
  const int64_t b = (total + threads - 1) / threads;
  return (int)(b < 148 * 16 ? b : 148 * 16);
}

}  // namespace

// in_dtype: the element type of `x` (the 32-bit residual stream, or activations of the compute dtype).
KVAD_EXPORT int kvad_rmsnorm(int in_dtype, int out_dtype, const void* x, int64_t ld_in, const int* row_index, const void* w,
                             int w_f32, int unit_offset, void* out, int64_t ld_out, int n_rows, int width, float eps,
                             cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && ld_in >= width && ld_out >= width, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
#define KVAD_RMS(TI, TO)                                                                                                  \
  kvad_launch(rmsnorm_kernel<TI, TO>, grid, block, 0, stream, (const TI*)x, ld_in, row_index, w, w_f32, unit_offset, (TO*)out, \
              ld_out, n_rows, width, eps)
  if (in_dtype == KVAD_DTYPE_F32 && out_dtype == KVAD_DTYPE_F32) KVAD_RMS(float, float);
  else if (in_dtype == KVAD_DTYPE_F32 && out_dtype == KVAD_DTYPE_BF16) KVAD_RMS(float, __nv_bfloat16);
  else if (in_dtype == KVAD_DTYPE_BF16 && out_dtype == KVAD_DTYPE_BF16) KVAD_RMS(__nv_bfloat16, __nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "rmsnorm: no form for input dtype %d and output dtype %d", in_dtype, out_dtype);
#undef KVAD_RMS
  KVAD_CHECK_LAUNCH("rmsnorm");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_residual_rmsnorm(int out_dtype, float* x, float* delta, float mult, int write_back, const int* row_index,
                                      const void* w, int w_f32, int unit_offset, void* out, int64_t ld_out, int n_rows,
                                      int width, float eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && ld_out >= width && x != nullptr && delta != nullptr, "residual_rmsnorm: bad arguments");
  KVAD_REQUIRE(!(write_back && row_index), "residual_rmsnorm: writing back goes with walking all rows");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
  const int vec = (width % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta)) & 15) == 0) ? 1 : 0;
  if (out_dtype == KVAD_DTYPE_F32)
    kvad_launch(residual_rmsnorm_kernel<float>, grid, block, 0, stream, x, delta, mult, write_back, row_index, w, w_f32, unit_offset,
                (float*)out, ld_out, n_rows, width, eps, vec);
  else if (out_dtype == KVAD_DTYPE_BF16)
    kvad_launch(residual_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, x, delta, mult, write_back, row_index, w, w_f32,
                unit_offset, (__nv_bfloat16*)out, ld_out, n_rows, width, eps, vec);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "residual_rmsnorm: unknown dtype %d", out_dtype);
  KVAD_CHECK_LAUNCH("residual_rmsnorm");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_scale_add(float* x, float* delta, float mult, int64_t total, cudaStream_t stream) {
  KVAD_REQUIRE(total >= 0 && x != nullptr && delta != nullptr, "scale_add: bad arguments");
  if (total == 0) return KVAD_OK;
  kvad_launch(scale_add_kernel, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, x, delta, mult, total);
  KVAD_CHECK_LAUNCH("scale_add");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_rotary(int dtype, const void* src, int64_t ld_src, int head_stride_src, int off_src, void* dst,
                            int64_t ld_dst, int head_stride_dst, int off_dst, const int* row_pos, const float* inv_freq,
                            int n_rows, int n_heads, int dims, int interleaved, int inverse, const void* head_gate,
                            int64_t ld_gate, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && dims > 0 && dims % 2 == 0, "rotary: bad sizes rows=%d heads=%d dims=%d", n_rows, n_heads, dims);
  KVAD_REQUIRE(row_pos != nullptr && inv_freq != nullptr, "rotary: needs positions and frequencies");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * n_heads * (dims / 2);
  dim3 grid(flat_blocks(total, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(rotary_kernel<float>, grid, block, 0, stream, (const float*)src, ld_src, head_stride_src, off_src, (float*)dst, ld_dst,
                head_stride_dst, off_dst, row_pos, inv_freq, n_rows, n_heads, dims, interleaved, inverse, (const float*)head_gate, ld_gate);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(rotary_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)src, ld_src, head_stride_src, off_src,
                (__nv_bfloat16*)dst, ld_dst, head_stride_dst, off_dst, row_pos, inv_freq, n_rows, n_heads, dims, interleaved, inverse,
                (const __nv_bfloat16*)head_gate, ld_gate);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "rotary: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("rotary");
  return KVAD_OK;
}

// act: 0 = silu, 1 = sigmoid, 2 = relu, 3 = the tanh form of GELU.
KVAD_EXPORT int kvad_gate_mul(int dtype, const void* a, int64_t ld_a, const void* b, int64_t ld_b, void* out, int64_t ld_out,
                              int n_rows, int width, int act, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && act >= 0 && act <= 3, "gate_mul: bad arguments rows=%d width=%d act=%d", n_rows, width, act);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(gate_mul_kernel<float>, grid, block, 0, stream, (const float*)a, ld_a, (const float*)b, ld_b, (float*)out, ld_out, n_rows, width, act);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(gate_mul_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)a, ld_a, (const __nv_bfloat16*)b, ld_b,
                (__nv_bfloat16*)out, ld_out, n_rows, width, act);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "gate_mul: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("gate_mul");
  return KVAD_OK;
}

// out null: only x += g * delta / rms(delta) (and delta = 0).
KVAD_EXPORT int kvad_postnorm_rmsnorm(int out_dtype, float* x, float* delta, const float* g, float eps_post, int write_back,
                                      const int* row_index, const void* w, int w_f32, int unit_offset, void* out, int64_t ld_out,
                                      int n_rows, int width, float eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && x != nullptr && delta != nullptr && g != nullptr, "postnorm_rmsnorm: bad arguments");
  KVAD_REQUIRE(!(write_back && row_index), "postnorm_rmsnorm: writing back goes with walking all rows");
  KVAD_REQUIRE(out == nullptr || ld_out >= width, "postnorm_rmsnorm: the output's rows are too short");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
  const bool few = n_rows <= 4 * 148 && width <= 128 * 16;
  if (out_dtype == KVAD_DTYPE_F32 && few)
    kvad_launch(postnorm_rmsnorm_kernel<float, true>, grid, block, 0, stream, x, delta, g, eps_post, write_back, row_index, w, w_f32, unit_offset,
                (float*)out, ld_out, width, eps);
  else if (out_dtype == KVAD_DTYPE_F32)
    kvad_launch(postnorm_rmsnorm_kernel<float, false>, grid, block, 0, stream, x, delta, g, eps_post, write_back, row_index, w, w_f32, unit_offset,
                (float*)out, ld_out, width, eps);
  else if (out_dtype == KVAD_DTYPE_BF16 && few)
    kvad_launch(postnorm_rmsnorm_kernel<__nv_bfloat16, true>, grid, block, 0, stream, x, delta, g, eps_post, write_back, row_index, w, w_f32,
                unit_offset, (__nv_bfloat16*)out, ld_out, width, eps);
  else if (out_dtype == KVAD_DTYPE_BF16)
    kvad_launch(postnorm_rmsnorm_kernel<__nv_bfloat16, false>, grid, block, 0, stream, x, delta, g, eps_post, write_back, row_index, w, w_f32,
                unit_offset, (__nv_bfloat16*)out, ld_out, width, eps);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "postnorm_rmsnorm: unknown dtype %d", out_dtype);
  KVAD_CHECK_LAUNCH("postnorm_rmsnorm");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_head_gate(int dtype, void* x, int64_t ld_x, const void* gate, int64_t ld_gate, int n_rows, int n_heads, int dv,
                               cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && dv > 0 && x && gate, "head_gate: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * n_heads * dv, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32) kvad_launch(head_gate_kernel<float>, grid, block, 0, stream, (float*)x, ld_x, (const float*)gate, ld_gate, n_rows, n_heads, dv);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(head_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)gate, ld_gate, n_rows, n_heads, dv);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "head_gate: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("head_gate");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_stream_concat(int dtype, const float* x, const float* x0, void* out, int n_rows, int width, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && x && x0 && out, "stream_concat: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32) kvad_launch(stream_concat_kernel<float>, grid, block, 0, stream, x, x0, (float*)out, n_rows, width);
  else if (dtype == KVAD_DTYPE_BF16) kvad_launch(stream_concat_kernel<__nv_bfloat16>, grid, block, 0, stream, x, x0, (__nv_bfloat16*)out, n_rows, width);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "stream_concat: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("stream_concat");
  return KVAD_OK;
}

// rows: a list of stream rows (n_rows of them) or null (the first n_rows).
KVAD_EXPORT int kvad_cast_rows(int out_dtype, const float* x, const int* row_index, void* out, int64_t ld_out, int n_rows, int width,
                               cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && x && out && ld_out >= width, "cast_rows: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (width % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (out_dtype == KVAD_DTYPE_F32 || out_dtype == KVAD_DTYPE_BF16)) {
    dim3 grid4(flat_blocks((int64_t)n_rows * (width / 4), 256));
    if (out_dtype == KVAD_DTYPE_F32) kvad_launch(cast_rows_vec_kernel<float>, grid4, block, 0, stream, x, row_index, (float*)out, ld_out, n_rows, width);
    else kvad_launch(cast_rows_vec_kernel<__nv_bfloat16>, grid4, block, 0, stream, x, row_index, (__nv_bfloat16*)out, ld_out, n_rows, width);
    KVAD_CHECK_LAUNCH("cast_rows");
    return KVAD_OK;
  }
  if (out_dtype == KVAD_DTYPE_F32) kvad_launch(cast_rows_kernel<float>, grid, block, 0, stream, x, row_index, (float*)out, ld_out, n_rows, width);
  else if (out_dtype == KVAD_DTYPE_BF16)
    kvad_launch(cast_rows_kernel<__nv_bfloat16>, grid, block, 0, stream, x, row_index, (__nv_bfloat16*)out, ld_out, n_rows, width);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "cast_rows: unknown dtype %d", out_dtype);
  KVAD_CHECK_LAUNCH("cast_rows");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_pair_norm_sum(float* a, float* b, const float* ga, const float* gb, float* delta, int n_rows, int width, float eps,
                                   float mult, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && a && b && ga && gb && delta, "pair_norm_sum: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  kvad_launch(pair_norm_sum_kernel, dim3(n_rows), dim3(128), 0, stream, a, b, ga, gb, delta, width, eps, mult);
  KVAD_CHECK_LAUNCH("pair_norm_sum");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_tanh_cap(float* x, int64_t total, float cap, cudaStream_t stream) {
  KVAD_REQUIRE(total >= 0 && x && cap > 0.f, "tanh_cap: bad arguments");
  if (total == 0) return KVAD_OK;
  kvad_launch(tanh_cap_kernel, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, x, total, cap);
  KVAD_CHECK_LAUNCH("tanh_cap");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
