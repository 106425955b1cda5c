// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        (S: [dk, dv] per sequence and head, 32-bit, kept in the cache)
//   o_t = S_t^T q_t
//
// with q and k turned by the row's position first (rotary, pairs half apart or interleaved, over the first
// `rot_dims` entries; angles, sines and the turned values in 32-bit), k scaled by `k_scale` after turning,
// and the output optionally divided by its root mean square per head and multiplied by silu(gate) where it
// is written.  Everything after the projections runs in 32-bit.  With `act` q, k and v pass a silu where they are
// staged (linear attention behind silu), and with `finish` off the raw 32-bit read-outs are all the kernel leaves:
// `row_norm_gate` then norms all heads of a row together, with a weight, times sigmoid(gate).
//
// A block owns one (sequence, head, range of value columns) - the columns of the state are independent of one
// another - and walks the sequence's rows of this step in order, 16 at a time: the block turns and stages the 16
// rows' q, k (one sine and cosine per pair, shared by q and k) and v in shared memory, then every thread carries
// its share of the state through them: thread (c, s) holds S[s * DPT .. s * DPT + DPT - 1][2c .. 2c + 1] in
// registers, the `split` threads of a column pair are neighbouring lanes and meet by shuffles.  Where one block
// has all columns of a head, it also divides the outputs by their root mean square and applies the gate; where
// a head's columns are spread over blocks, the raw 32-bit outputs go to `raw` and a second kernel finishes them.
// A single-token row is the same walk with one row, so decoding and prompts (whole or in portions) give the
// same bits.  The state is read from the sequence's slot at the start and written back at the end.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int TB = 16, VPT = 2;

struct RetentionArgs {
  const void* q; const void* k; const void* v; const void* gate;
  int64_t ld_q, ld_k, ld_v, ld_gate;
  void* out; int64_t ld_out;
  float* raw;                           // [rows, heads * dv], used when a head's columns are spread over blocks
  float* state;                         // [slots, heads, dk, dv]
  const int* seq_starts; const int* kv_lens; const int* seq_slots;
  const float* decay;                   // [heads]
  const float* inv_freq;                // [rot_dims / 2] or null
  int rot_dims, interleaved;
  int heads, dk, dv, split, vc, fused, vec;
  float k_scale, eps;
  int unit_norm;
  int act;                              // 1: q, k and v pass a silu as they are staged
  int finish;                           // 0: only the raw 32-bit read-outs are written (to `raw`)
};

__device__ __forceinline__ void unpack16(const uint4& raw, float* f, float) {
  f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void unpack16(const uint4& raw, float* f, __nv_bfloat16) {
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 v = __bfloat1622float2(h2[t]);
    f[2 * t] = v.x;
    f[2 * t + 1] = v.y;
  }
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__device__ __forceinline__ void finish_row(const float* o, int dv, int lane, bool unit_norm, float eps, const T* gate, T* out) {
  float inv = 1.f;
  if (unit_norm) {
    float sq = 0.f;
    for (int c = lane; c < dv; c += 32) sq = fmaf(o[c], o[c], sq);
    sq = warp_sum(sq);
    inv = 1.0f / sqrtf(sq / (float)dv + eps);
  }
  for (int c = lane; c < dv; c += 32) {
    float y = o[c] * inv;
    if (gate != nullptr) {
      const float g = to_f32(gate[c]);
      y *= g / (1.0f + expf(-g));
    }
    out[c] = from_f32<T>(y);
  }
}

template <typename T, int DPT>
__global__ void __launch_bounds__(256) retention_kernel(const RetentionArgs a) {
  extern __shared__ float smem[];
  // (a thread's DPT entries are followed by 4 floats of padding, so that the `split` lanes of a column pair read
  // different banks with their 16-byte loads)
  constexpr int SEG = DPT + 4;
  const int dk = a.dk, dv = a.dv, split = a.split, dkp = split * DPT, lds = split * SEG, vc = a.vc;
  float* qs = smem;                     // [TB][split][SEG]
  float* ks = qs + TB * lds;            // [TB][split][SEG]
  float* vs = ks + TB * lds;            // [TB][vc]
  float* os = vs + TB * vc;             // [TB][vc]
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, v_base = blockIdx.z * vc, tid = threadIdx.x, nthreads = blockDim.x;
  const int start = a.seq_starts[s], n_new = a.seq_starts[s + 1] - start;
  const int pos0 = a.kv_lens[s] - n_new;
  const int ci = tid / split, si = tid - ci * split;               // column pair, share of the key entries
  const int c0 = ci * VPT;                                          // first of the thread's columns, within the block's range
  const bool own0 = c0 < vc && v_base + c0 < dv, own1 = c0 + 1 < vc && v_base + c0 + 1 < dv;
  float* st = a.state + ((int64_t)a.seq_slots[s] * a.heads + h) * dk * dv;
  const float decay = a.decay[h];
  float S0[DPT], S1[DPT];
#pragma unroll
  for (int j = 0; j < DPT; ++j) {
    const int d = si * DPT + j;
    S0[j] = (own0 && d < dk) ? st[(int64_t)d * dv + v_base + c0] : 0.f;
    S1[j] = (own1 && d < dk) ? st[(int64_t)d * dv + v_base + c0 + 1] : 0.f;
  }
  const T* q = (const T*)a.q;
  const T* k = (const T*)a.k;
  const T* v = (const T*)a.v;
  const T* gate = (const T*)a.gate;
  T* out = (T*)a.out;
  const int half = a.inv_freq != nullptr ? a.rot_dims / 2 : 0;
  // The rows of the batch after this one are fetched into registers, in 16-byte pieces, while this one is worked
  // (`a.vec`: sizes, strides and addresses allow the pieces; up to NP pieces of q and of k a thread, one of v);
  // otherwise the rows are fetched entry by entry where they are stored.
  constexpr int E = 16 / (int)sizeof(T), NP = 4;
  const int cpr = dkp / E, vpr = vc / E;                         // pieces of a row of q / k, of v
  const bool ahead = a.vec != 0 && TB * cpr <= NP * nthreads && TB * vpr <= nthreads;
  uint4 q_pf[NP], k_pf[NP], v_pf;
  auto fetch = [&](int t0) {
    const int nb = n_new - t0 < TB ? n_new - t0 : TB;
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      const int i = tid + u * nthreads, t = i / cpr, c = (i - t * cpr) * E;
      q_pf[u] = k_pf[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < nb * cpr && c < dk) {
        const int64_t row = start + t0 + t;
        q_pf[u] = *reinterpret_cast<const uint4*>(q + row * a.ld_q + (int64_t)h * dk + c);
        k_pf[u] = *reinterpret_cast<const uint4*>(k + row * a.ld_k + (int64_t)h * dk + c);
      }
    }
    const int t = tid / vpr, c = (tid - t * vpr) * E;
    v_pf = make_uint4(0u, 0u, 0u, 0u);
    if (tid < nb * vpr && v_base + c < dv) v_pf = *reinterpret_cast<const uint4*>(v + (int64_t)(start + t0 + t) * a.ld_v + (int64_t)h * dv + v_base + c);
  };
  if (ahead && n_new > 0) fetch(0);
  for (int t0 = 0; t0 < n_new; t0 += TB) {
    const int nb = n_new - t0 < TB ? n_new - t0 : TB;
    __syncthreads();                                            // the rows before have been used up
    // raw rows first, then the pairs are turned where they lie
    if (ahead) {
#pragma unroll
      for (int u = 0; u < NP; ++u) {
        const int i = tid + u * nthreads, t = i / cpr, c = (i - t * cpr) * E;
        if (i < nb * cpr) {
          float fq[E], fk[E];
          unpack16(q_pf[u], fq, T());
          unpack16(k_pf[u], fk, T());
          if (a.act) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
              fq[e] = c + e < dk ? silu_f(fq[e]) : 0.f;
              fk[e] = c + e < dk ? silu_f(fk[e]) : 0.f;
            }
          }
#pragma unroll
          for (int e = 0; e < E; ++e) fk[e] *= (c + e < 2 * half ? 1.f : a.k_scale);      // (turned entries are scaled after turning)
          float* qd = qs + t * lds + (c / DPT) * SEG + c % DPT;
          float* kd = ks + t * lds + (c / DPT) * SEG + c % DPT;
#pragma unroll
          for (int e = 0; e < E; e += 4) {
            *reinterpret_cast<float4*>(qd + e) = make_float4(fq[e], fq[e + 1], fq[e + 2], fq[e + 3]);
            *reinterpret_cast<float4*>(kd + e) = make_float4(fk[e], fk[e + 1], fk[e + 2], fk[e + 3]);
          }
        }
      }
      if (tid < nb * vpr) {
        float fv[E];
        unpack16(v_pf, fv, T());
        if (a.act) {
#pragma unroll
          for (int e = 0; e < E; ++e) fv[e] = silu_f(fv[e]);
        }
#pragma unroll
        for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(vs + tid * E + e) = make_float4(fv[e], fv[e + 1], fv[e + 2], fv[e + 3]);
      }
      if (t0 + TB < n_new) fetch(t0 + TB);                      // in flight while this batch is turned and walked
    } else {
#pragma unroll 4
      for (int i = tid; i < nb * dkp; i += nthreads) {
        const int t = i / dkp, d = i - t * dkp, at = t * lds + (d / DPT) * SEG + d % DPT;
        const int64_t row = start + t0 + t;
        float qv = d < dk ? to_f32(q[row * a.ld_q + (int64_t)h * dk + d]) : 0.f;
        float kv = d < dk ? to_f32(k[row * a.ld_k + (int64_t)h * dk + d]) : 0.f;
        if (a.act) {
          qv = silu_f(qv);
          kv = silu_f(kv);
        }
        qs[at] = qv;
        ks[at] = kv * (d < 2 * half ? 1.f : a.k_scale);
      }
#pragma unroll 4
      for (int i = tid; i < nb * vc; i += nthreads) {
        const int t = i / vc, c = i - t * vc;
        float vv = v_base + c < dv ? to_f32(v[(int64_t)(start + t0 + t) * a.ld_v + (int64_t)h * dv + v_base + c]) : 0.f;
        vs[i] = a.act ? silu_f(vv) : vv;
      }
    }
    if (half > 0) {
      __syncthreads();
      for (int i = tid; i < nb * half; i += nthreads) {         // one sine and cosine per pair, for q and k
        const int t = i / half, p = i - t * half;
        const int ea = a.interleaved ? 2 * p : p, eb = a.interleaved ? 2 * p + 1 : p + half;
        const int da = t * lds + (ea / DPT) * SEG + ea % DPT, db = t * lds + (eb / DPT) * SEG + eb % DPT;
        float sn, cs;
        sincosf((float)(pos0 + t0 + t) * a.inv_freq[p], &sn, &cs);
        const float qa = qs[da], qb = qs[db], ka = ks[da], kb = ks[db];
        qs[da] = qa * cs - qb * sn;
        qs[db] = qb * cs + qa * sn;
        ks[da] = (ka * cs - kb * sn) * a.k_scale;
        ks[db] = (kb * cs + ka * sn) * a.k_scale;
      }
    }
    __syncthreads();
    if ((tid & ~31) < (vc / VPT) * split) {                     // (whole warps walk, also a thread without columns: the shuffles want them; the other warps only stage)
      // four rows at a time: their loads and multiply-adds first (only the state links them), then the lanes' sums
      // of all four meet by shuffles side by side, then the stores - so that no row waits for the one before it
      for (int tb = 0; tb < nb; tb += 4) {
        float r0[4], r1[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int t = tb + w;
          r0[w] = r1[w] = 0.f;
          if (t < nb) {                                         // (the same for the whole block)
            const float v0 = c0 < vc ? vs[t * vc + c0] : 0.f, v1 = c0 + 1 < vc ? vs[t * vc + c0 + 1] : 0.f;
            const float4* kt = reinterpret_cast<const float4*>(ks + t * lds + si * SEG);
            const float4* qt = reinterpret_cast<const float4*>(qs + t * lds + si * SEG);
            float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j4 = 0; j4 < DPT / 4; ++j4) {
              const float4 kk = kt[j4], qq = qt[j4];
              const float kj[4] = {kk.x, kk.y, kk.z, kk.w}, qj[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int j = j4 * 4 + u;
                S0[j] = fmaf(kj[u], v0, decay * S0[j]);
                S1[j] = fmaf(kj[u], v1, decay * S1[j]);
                o0[u] = fmaf(S0[j], qj[u], o0[u]);
                o1[u] = fmaf(S1[j], qj[u], o1[u]);
              }
            }
            r0[w] = (o0[0] + o0[1]) + (o0[2] + o0[3]);
            r1[w] = (o1[0] + o1[1]) + (o1[2] + o1[3]);
          }
        }
        for (int m = 1; m < split; m <<= 1) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            r0[w] += __shfl_xor_sync(0xffffffffu, r0[w], m);
            r1[w] += __shfl_xor_sync(0xffffffffu, r1[w], m);
          }
        }
        if (si == 0 && c0 < vc) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            if (tb + w < nb) {
              os[(tb + w) * vc + c0] = r0[w];
              if (c0 + 1 < vc) os[(tb + w) * vc + c0 + 1] = r1[w];
            }
          }
        }
      }
    }
    __syncthreads();
    if (a.fused) {          // the block has the head's columns: a warp per row finishes it
      for (int t = tid >> 5; t < nb; t += nthreads >> 5) {
        const int64_t row = start + t0 + t;
        finish_row<T>(os + t * vc, dv, tid & 31, a.unit_norm != 0, a.eps, gate ? gate + row * a.ld_gate + (int64_t)h * dv : nullptr,
                      out + row * a.ld_out + (int64_t)h * dv);
      }
    } else {
      for (int i = tid; i < nb * vc; i += nthreads) {
        const int t = i / vc, c = i - t * vc;
        if (v_base + c < dv) a.raw[(int64_t)(start + t0 + t) * a.heads * dv + (int64_t)h * dv + v_base + c] = os[i];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < DPT; ++j) {
    const int d = si * DPT + j;
    if (own0 && d < dk) st[(int64_t)d * dv + v_base + c0] = S0[j];
    if (own1 && d < dk) st[(int64_t)d * dv + v_base + c0 + 1] = S1[j];
  }
}

// A warp per (row, head): raw outputs over their root mean square, times silu(gate), stored.
template <typename T>
__global__ void __launch_bounds__(128)
retention_finish_kernel(const float* __restrict__ raw, int n_rows, int heads, int dv, int unit_norm, float eps,
                        const T* __restrict__ gate, int64_t ld_gate, T* __restrict__ out, int64_t ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (int64_t)n_rows * heads) return;
  const int64_t row = item / heads;
  const int h = (int)(item % heads);
  finish_row<T>(raw + row * heads * dv + (int64_t)h * dv, dv, threadIdx.x & 31, unit_norm != 0, eps,
                gate ? gate + row * ld_gate + (int64_t)h * dv : nullptr, out + row * ld_out + (int64_t)h * dv);
}

// out = raw / sqrt(mean over the whole row (raw^2) + eps) * w * sigmoid(gate): a block per row of 32-bit read-outs.
template <typename T>
__global__ void __launch_bounds__(128)
row_norm_gate_kernel(const float* __restrict__ raw, int64_t ld_raw, const T* __restrict__ gate, int64_t ld_gate, const void* __restrict__ w,
                     int w_f32, T* __restrict__ out, int64_t ld_out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* o = raw + (int64_t)blockIdx.x * ld_raw;
  float sq = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) sq = fmaf(o[c], o[c], sq);
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    float y = o[c] * inv;
    if (w != nullptr) y *= load_param(w, c, w_f32);
    if (gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(gate[(int64_t)blockIdx.x * ld_gate + c])));
    out[(int64_t)blockIdx.x * ld_out + c] = from_f32<T>(y);
  }
}

// How the state of a head is spread: a thread holds DPT key entries of two columns - 8 of them, so that the walk
// over a row is short (a head of 128 key entries: 16 lanes a column pair), more only where 32 lanes are not enough -
// and the threads that carry state are at most 128 a block and hold at most 32 columns (more blocks rather than
// wider ones) unless that is the whole head.
struct Spread { int dpt, split, vc, fused; };
inline Spread spread_of(int dk, int dv) {
  int p2 = 8;
  while (p2 < dk) p2 <<= 1;
  Spread z;
  z.split = p2 / 8 > 32 ? 32 : p2 / 8;
  z.dpt = p2 / z.split;
  const int fit = z.split <= 32 ? VPT * (128 / z.split) : 0;
  z.vc = fit >= dv ? (dv + VPT - 1) / VPT * VPT : (fit > 32 ? 32 : fit);
  z.fused = z.vc >= dv ? 1 : 0;
  return z;
}

template <typename T, int DPT>
int launch_retention(const RetentionArgs& a, int n_seqs, int n_rows, cudaStream_t stream) {
  const size_t smem = ((size_t)2 * TB * a.split * (DPT + 4) + (size_t)2 * TB * a.vc) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(retention_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "retention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  // (a block of 256 threads: the first (vc / 2) * split carry the state, all of them stage the rows; single-token rows need no helpers)
  const int threads = n_rows > n_seqs ? 256 : ((a.vc / VPT) * a.split + 31) / 32 * 32;
  kvad_launch(retention_kernel<T, DPT>, dim3(n_seqs, a.heads, (a.dv + a.vc - 1) / a.vc), dim3(threads), smem, stream, a);
  KVAD_CHECK_LAUNCH("retention");
  if (!a.fused && a.finish) {
    const int64_t items = (int64_t)n_rows * a.heads;
    kvad_launch(retention_finish_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const float*)a.raw, n_rows, a.heads, a.dv,
                a.unit_norm, a.eps, (const T*)a.gate, a.ld_gate, (T*)a.out, a.ld_out);
    KVAD_CHECK_LAUNCH("retention (finish)");
  }
  return KVAD_OK;
}

template <typename T>
int dispatch_retention(RetentionArgs& a, int n_seqs, int n_rows, cudaStream_t stream) {
  const Spread z = spread_of(a.dk, a.dv);
  if (z.dpt > 32) KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "retention: keys of %d entries a head are above this kernel's limit of 1024", a.dk);
  a.split = z.split; a.vc = z.vc; a.fused = a.finish ? z.fused : 0;
  const int piece = 16 / (int)sizeof(T);                        // entries of a 16-byte piece
  a.vec = (a.dk % piece == 0 && a.dv % piece == 0 && a.vc % piece == 0 && a.ld_q % piece == 0 && a.ld_k % piece == 0 && a.ld_v % piece == 0 &&
           ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) == 0) ? 1 : 0;
  if (!a.fused && a.raw == nullptr) KVAD_FAIL(KVAD_ERR_ARGUMENT, "retention: heads of %d value columns need the 32-bit scratch", a.dv);
  switch (z.dpt) {
    case 8: return launch_retention<T, 8>(a, n_seqs, n_rows, stream);
    case 16: return launch_retention<T, 16>(a, n_seqs, n_rows, stream);
    default: return launch_retention<T, 32>(a, n_seqs, n_rows, stream);
  }
}

}  // namespace

// 1 if heads of this shape have their value columns spread over blocks, so that kvad_retention needs `raw`.
KVAD_EXPORT int kvad_retention_needs_raw(int dk, int dv) { return spread_of(dk, dv).fused ? 0 : 1; }

// `raw`: float32 [rows, heads * dv] (see kvad_retention_needs_raw), `n_rows`: the step's rows.
KVAD_EXPORT int kvad_retention(int dtype, const void* q, int64_t ld_q, const void* k, int64_t ld_k, const void* v, int64_t ld_v,
                               const void* gate, int64_t ld_gate, void* out, int64_t ld_out, float* raw, int n_rows, float* state, const int* seq_starts,
                               const int* kv_lens, const int* seq_slots, const float* decay, const float* inv_freq, int rot_dims,
                               int interleaved, int n_seqs, int heads, int dk, int dv, float k_scale, float eps, int unit_norm,
                               int act, int finish, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && heads > 0 && dk > 0 && dv > 0, "retention: bad sizes seqs=%d heads=%d dk=%d dv=%d", n_seqs, heads, dk, dv);
  KVAD_REQUIRE(state != nullptr && decay != nullptr && seq_starts && kv_lens && seq_slots, "retention: needs state, decays and the step's sequences");
  KVAD_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk, "retention: %d rotated entries of %d", rot_dims, dk);
  KVAD_REQUIRE(n_seqs <= 65535 * 32 && heads <= 65535, "retention: %d sequences x %d heads are more than one launch takes", n_seqs, heads);
  if (n_seqs == 0) return KVAD_OK;
  RetentionArgs a;
  a.q = q; a.k = k; a.v = v; a.gate = gate; a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_gate = ld_gate;
  a.out = out; a.ld_out = ld_out; a.raw = raw; a.vc = 0; a.fused = 1; a.vec = 0; a.state = state; a.seq_starts = seq_starts; a.kv_lens = kv_lens; a.seq_slots = seq_slots;
  a.decay = decay; a.inv_freq = rot_dims > 0 ? inv_freq : nullptr; a.rot_dims = rot_dims; a.interleaved = interleaved;
  a.heads = heads; a.dk = dk; a.dv = dv; a.split = 1; a.k_scale = k_scale; a.eps = eps; a.unit_norm = unit_norm; a.act = act ? 1 : 0; a.finish = finish ? 1 : 0;
  KVAD_REQUIRE(finish || raw != nullptr, "retention: raw read-outs need the 32-bit scratch");
  if (dtype == KVAD_DTYPE_F32) return dispatch_retention<float>(a, n_seqs, n_rows, stream);
  if (dtype == KVAD_DTYPE_BF16) return dispatch_retention<__nv_bfloat16>(a, n_seqs, n_rows, stream);
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "retention: unknown dtype %d", dtype);
}

// raw: float32 [rows, width]; gate, out: of `dtype`; w: `width` weights (float32 or bfloat16) or null.
KVAD_EXPORT int kvad_row_norm_gate(int dtype, const float* raw, int64_t ld_raw, const void* gate, int64_t ld_gate, const void* w, int w_f32,
                                   void* out, int64_t ld_out, int n_rows, int width, float eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && raw && out, "row_norm_gate: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(row_norm_gate_kernel<float>, dim3(n_rows), dim3(128), 0, stream, raw, ld_raw, (const float*)gate, ld_gate, w, w_f32, (float*)out, ld_out, width, eps);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(row_norm_gate_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, stream, raw, ld_raw, (const __nv_bfloat16*)gate, ld_gate, w, w_f32,
                (__nv_bfloat16*)out, ld_out, width, eps);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "row_norm_gate: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("row_norm_gate");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
