// Softmax attention over the paged cache with everything a score can be given on its way to the softmax,
// on the CUDA cores in 32-bit arithmetic, for prompts and for single-token rows alike:
//
//   s = (q . k) * scale;  s = cap * tanh(s / cap)  (cap > 0);  s -= slope_h * (i - j)  (slope_span > 0,
//   slope_h = 2^(-slope_span * (h + 1) / n_heads));  query i sees key j if j <= i and
//   (window <= 0 or i - j < window or j < keep_first).
//
// Keys and values may differ in size (dk, dv), several query heads may share a key/value head, and the
// values may BE the keys' first dv entries (`v_pages` = `k_pages` with the keys' row stride): a latent
// cache read by queries that were carried into the latent's space.  The output may be multiplied by
// sigmoid(gate) where it is written.
//
// A block works a tile of 32 (or, with eight warps, 64) (token, head) pairs that share one key/value head - 32 / hp consecutive
// tokens of one sequence times hp heads of the group (prompts: few heads, many tokens; single-token rows:
// one token, all heads of the group) - against the keys tile by tile: a tile of keys and values comes into
// shared memory once for all 32 pairs.  Warp w owns pairs 8w .. 8w+7: for the scores a lane takes keys
// lane (and lane + 32) of the tile for all eight, maxima and sums meet by shuffles, the weights go through
// shared memory, and for the output a lane owns dimensions lane, lane + 32, ...  Tiles of keys that no
// pair of the block sees (before every window and past the kept first tokens) are skipped, so pages that
// the cache has dropped are never touched.
//
// Also here: the cache writes that go with it - keys and values of different sizes with the values blended
// with another layer's (`kv_store_blend`), queries, keys and values turned by their positions and the keys and values
// stored in the same pass (`turn_store`), and a latent row normalised, its rotary part turned, and stored
// (`latent_store`).
//
// Several key heads may share one value head (`key_maps` consecutive key heads read value head kvh / key_maps): the maps
// of a differential attention are attentions of their own over the same values.  `diff_combine` then takes the second
// map off the first, o = a1 - lambda a2, and makes each head a unit vector by its root mean square.  `norm_turn_store`
// is `turn_store` for queries and keys that are RMS-normed first, head by head or over the whole projection, with a
// factor on cosine and sine (stretched frequencies).
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int RPW = 8, PAGE = 64;       // pairs a warp owns; a block of NW warps works 8 * NW pairs (4 warps: 32, 8 warps: 64)

struct ScoredArgs {
  const void* q; int64_t ld_q;
  void* out; int64_t ld_out;
  const void* gate; int64_t ld_gate;
  const int* seq_starts; const int* kv_lens; const int* page_table; int table_width;
  const void* k_pages; const void* v_pages;
  int64_t k_page_stride, k_head_stride, v_page_stride, v_head_stride;   // in elements
  int ld_k, ld_v;                                                       // row strides inside a page
  int n_heads, n_kv_heads, dk, dv, hp, v_alias;
  int key_maps;          // this many consecutive key heads read one value head
  int out_f32;           // the output is 32-bit whatever the storage type (no gate then)
  int merge;             // 0: with n_splits > 1 the parts are left in `partial` for a merge of the caller's
  float scale, softcap, slope_span;
  int window, keep_first;
  int vec_k, vec_v;      // keys / values can be fetched in 16-byte pieces
  int n_splits;          // > 1: the tiles of keys a block would walk are dealt out to n_splits blocks; each leaves its
  float* partial;        // running maximum, sum and unnormalised output in `partial` [rows, heads, n_splits, dv + 2]
};

__device__ __forceinline__ void unpack16(const uint4& raw, float* f, float) {
  f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void unpack16(const uint4& raw, float* f, __nv_bfloat16) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 v = __bfloat1622float2(h[t]);
    f[2 * t] = v.x;
    f[2 * t + 1] = v.y;
  }
}

// `n_rows` rows of `cols` entries (row stride ld_src) into 32-bit shared memory (row stride ld_dst, `cols_to` >= cols
// entries written, the rest zeros); rows from `n_live` on are zeros (places of the cache that no row sees yet may hold
// anything).  `vec`: 16-byte pieces (cols, ld_src multiples of a piece, src aligned) - few, wide, independent loads.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld_dst, const T* src, int64_t ld_src, int n_rows, int cols, int cols_to,
                                          int n_live, bool vec, int tid, int nthreads) {
  constexpr int E = 16 / (int)sizeof(T);
  if (vec) {
    const int cpr = cols / E;
#pragma unroll 4
    for (int i = tid; i < n_rows * cpr; i += nthreads) {
      const int r = i / cpr, c = (i - r * cpr) * E;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (r < n_live) raw = *reinterpret_cast<const uint4*>(src + (int64_t)r * ld_src + c);
      float f[E];
      unpack16(raw, f, T());
#pragma unroll
      for (int e = 0; e < E; ++e) dst[r * ld_dst + c + e] = f[e];
    }
    for (int i = tid; i < n_rows * (cols_to - cols); i += nthreads) {
      const int r = i / (cols_to - cols), c = cols + (i - r * (cols_to - cols));
      dst[r * ld_dst + c] = 0.f;
    }
  } else {
#pragma unroll 4
    for (int i = tid; i < n_rows * cols_to; i += nthreads) {
      const int r = i / cols_to, c = i - r * cols_to;
      dst[r * ld_dst + c] = (r < n_live && c < cols) ? to_f32(src[(int64_t)r * ld_src + c]) : 0.f;
    }
  }
}

template <typename T, int KPL, int DPL, int NW>
__global__ void __launch_bounds__(32 * NW) scored_attention_kernel(const ScoredArgs a) {
  constexpr int TK = 32 * KPL, TR = RPW * NW, THREADS = 32 * NW;
  extern __shared__ float smem[];
  const int dk = a.dk, dv = a.dv, dkp = (dk + 3) & ~3, ldks = dkp + 1, ldvs = a.v_alias ? ldks : dv;   // (keys padded with zeros to fours)
  float* Qs = smem;                                   // [TR][dkp]
  float* Ks = Qs + TR * dkp;                          // [TK][dkp + 1]
  float* Vs = a.v_alias ? Ks : Ks + TK * ldks;        // [TK][ldvs]
  float* Ps = a.v_alias ? Ks + TK * ldks : Vs + TK * dv;   // [TR][TK]
  pdl_launch_dependents();
  pdl_wait();
  const int hp = a.hp, tok = TR / hp;
  const int group = a.n_heads / a.n_kv_heads, chunks = (group + hp - 1) / hp;
  const int s = blockIdx.y, kvh = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
  const int n_splits = a.n_splits, split = blockIdx.x % n_splits;
  const int start = a.seq_starts[s], n_new = a.seq_starts[s + 1] - start, tok0 = (blockIdx.x / n_splits) * tok;
  if (tok0 >= n_new) return;
  const int n_tok = n_new - tok0 < tok ? n_new - tok0 : tok;
  const int h0 = kvh * group + chunk * hp, n_h = group - chunk * hp < hp ? group - chunk * hp : hp;
  const int pos0 = a.kv_lens[s] - n_new + tok0, last_pos = pos0 + n_tok - 1;
  const int* pages = a.page_table + (int64_t)s * a.table_width;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* q = (const T*)a.q;

  for (int i = tid; i < TR * dkp; i += THREADS) {
    const int r = i / dkp, d = i - r * dkp, ti = r / hp, hi = r - ti * hp;
    Qs[i] = (ti < n_tok && hi < n_h && d < dk) ? to_f32(q[(int64_t)(start + tok0 + ti) * a.ld_q + (int64_t)(h0 + hi) * dk + d]) : 0.f;
  }
  // what each of the warp's pairs is: its position, whether it exists, its head's slope
  int row_pos[RPW];
  bool row_live[RPW], warp_live = false;
  float row_slope[RPW];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int row = warp * RPW + r, ti = row / hp, hi = row - ti * hp;
    row_live[r] = ti < n_tok && hi < n_h;
    warp_live = warp_live || row_live[r];
    row_pos[r] = pos0 + ti;
    row_slope[r] = a.slope_span > 0.f ? exp2f(-a.slope_span * (float)(h0 + hi + 1) / (float)a.n_heads) : 0.f;
  }
  float acc[RPW][DPL], run_max[RPW], run_sum[RPW];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    run_max[r] = -INFINITY;
    run_sum[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
  }
  const int first_key = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;   // of the block's first token
  const T* kp = (const T*)a.k_pages;
  const T* vp = (const T*)a.v_pages;
  int dealt = 0;
  for (int t = 0; t <= last_pos / TK; ++t) {
    const int key0 = t * TK;
    if (key0 + TK <= first_key && key0 >= a.keep_first) continue;       // (the same for every thread of the block)
    if (dealt++ % n_splits != split) continue;
    __syncthreads();                                                    // the tile before has been used up (and Qs is written)
    const int page = pages[key0 / PAGE], in_page = key0 % PAGE;
    const T* kt = kp + (int64_t)page * a.k_page_stride + (int64_t)kvh * a.k_head_stride + (int64_t)in_page * a.ld_k;
    const int n_live = last_pos - key0 + 1;                             // keys of the tile that exist
    load_tile<T>(Ks, ldks, kt, a.ld_k, TK, dk, dkp, n_live, a.vec_k != 0, tid, THREADS);
    if (!a.v_alias) {
      const T* vt = vp + (int64_t)page * a.v_page_stride + (int64_t)(kvh / a.key_maps) * a.v_head_stride + (int64_t)in_page * a.ld_v;
      load_tile<T>(Vs, dv, vt, a.ld_v, TK, dv, dv, n_live, a.vec_v != 0, tid, THREADS);
    }
    __syncthreads();
    if (!warp_live) continue;                                           // (a warp without pairs only helps to load)
    float sc[RPW][KPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int j = 0; j < KPL; ++j) sc[r][j] = 0.f;
    const float* qw = Qs + warp * RPW * dkp;
    for (int d = 0; d < dkp; d += 4) {
      float kv[KPL][4];
#pragma unroll
      for (int j = 0; j < KPL; ++j) {
        const float* kr = Ks + (lane + 32 * j) * ldks + d;
        kv[j][0] = kr[0]; kv[j][1] = kr[1]; kv[j][2] = kr[2]; kv[j][3] = kr[3];
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float4 qv = *reinterpret_cast<const float4*>(qw + r * dkp + d);
#pragma unroll
        for (int j = 0; j < KPL; ++j)
          sc[r][j] = fmaf(qv.w, kv[j][3], fmaf(qv.z, kv[j][2], fmaf(qv.y, kv[j][1], fmaf(qv.x, kv[j][0], sc[r][j]))));
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int pos = row_pos[r];
      float v[KPL];
      float tile_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < KPL; ++j) {
        const int key = key0 + lane + 32 * j;
        v[j] = -INFINITY;
        if (row_live[r] && key <= pos && (a.window <= 0 || pos - key < a.window || key < a.keep_first)) {
          float x = sc[r][j] * a.scale;
          if (a.softcap > 0.f) x = a.softcap * tanhf(x / a.softcap);
          v[j] = x - row_slope[r] * (float)(pos - key);
        }
        tile_max = fmaxf(tile_max, v[j]);
      }
      tile_max = warp_max(tile_max);
      const float new_max = fmaxf(run_max[r], tile_max);
      const float base = new_max == -INFINITY ? 0.f : new_max;
      const float keep = run_max[r] == -INFINITY ? 0.f : expf(run_max[r] - base);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < KPL; ++j) {
        const float p = v[j] == -INFINITY ? 0.f : expf(v[j] - base);
        Ps[(warp * RPW + r) * TK + lane + 32 * j] = p;
        psum += p;
      }
      run_sum[r] = run_sum[r] * keep + warp_sum(psum);
      run_max[r] = new_max;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[r][i] *= keep;
    }
    __syncwarp();
    const float* pw = Ps + warp * RPW * TK;
    for (int k = 0; k < TK; k += 4) {
      float4 pv[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) pv[r] = *reinterpret_cast<const float4*>(pw + r * TK + k);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) {
          const float x0 = Vs[k * ldvs + d], x1 = Vs[(k + 1) * ldvs + d], x2 = Vs[(k + 2) * ldvs + d], x3 = Vs[(k + 3) * ldvs + d];
#pragma unroll
          for (int r = 0; r < RPW; ++r)
            acc[r][i] = fmaf(pv[r].w, x3, fmaf(pv[r].z, x2, fmaf(pv[r].y, x1, fmaf(pv[r].x, x0, acc[r][i]))));
        }
      }
    }
  }
  T* out = (T*)a.out;
  const T* gate = (const T*)a.gate;
  if (n_splits > 1) {
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      if (!row_live[r]) continue;
      const int row = warp * RPW + r, ti = row / hp, hi = row - ti * hp;
      float* dst = a.partial + (((int64_t)(start + tok0 + ti) * a.n_heads + h0 + hi) * n_splits + split) * (dv + 2);
      if (lane == 0) {
        dst[0] = run_max[r];
        dst[1] = run_sum[r];
      }
#pragma unroll
      for (int i = 0; i < DPL; ++i)
        if (lane + 32 * i < dv) dst[2 + lane + 32 * i] = acc[r][i];
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    if (!row_live[r]) continue;
    const int row = warp * RPW + r, ti = row / hp, hi = row - ti * hp;
    const float inv = 1.0f / run_sum[r];
    const int64_t grow = start + tok0 + ti;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) {
        float y = acc[r][i] * inv;
        if (gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(gate[grow * a.ld_gate + (int64_t)(h0 + hi) * dv + d])));
        if (a.out_f32) reinterpret_cast<float*>(a.out)[grow * a.ld_out + (int64_t)(h0 + hi) * dv + d] = y;
        else out[grow * a.ld_out + (int64_t)(h0 + hi) * dv + d] = from_f32<T>(y);
      }
    }
  }
}

// The parts that `n_splits` blocks left of one (row, head) become its output: a block per (row, head), a thread per
// output entry; the parts are taken in split order, so the result does not depend on which block finished first.
template <typename T>
__global__ void scored_merge_kernel(const float* __restrict__ partial, int n_splits, int n_heads, int dv, T* __restrict__ out,
                                    int64_t ld_out, const T* __restrict__ gate, int64_t ld_gate, int out_f32) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, h = blockIdx.y;
  const float* src = partial + ((int64_t)row * n_heads + h) * n_splits * (dv + 2);
  float m = -INFINITY;
#pragma unroll 4
  for (int i = 0; i < n_splits; ++i) m = fmaxf(m, src[i * (dv + 2)]);
  float total = 0.f;
  for (int i = 0; i < n_splits; ++i) {
    const float mi = src[i * (dv + 2)];
    if (mi != -INFINITY) total = fmaf(src[i * (dv + 2) + 1], expf(mi - m), total);
  }
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float y = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float mi = src[i * (dv + 2)];
      if (mi != -INFINITY) y = fmaf(src[i * (dv + 2) + 2 + d], expf(mi - m), y);
    }
    y /= total;
    if (gate != nullptr) y *= 1.0f / (1.0f + expf(-to_f32(gate[(int64_t)row * ld_gate + (int64_t)h * dv + d])));
    if (out_f32) reinterpret_cast<float*>(out)[(int64_t)row * ld_out + (int64_t)h * dv + d] = y;
    else out[(int64_t)row * ld_out + (int64_t)h * dv + d] = from_f32<T>(y);
  }
}

// The same merge for the two maps of a differential attention, and its last step with it: a block per (row, head of the
// output) merges both maps' parts (`partial` rows are laid out [kv head][map][head of the group]), takes the second map
// off the first with `lambda`, and writes o * gain / sqrt(mean(o^2) + eps).  A thread per value entry.
template <typename T>
__global__ void __launch_bounds__(128)
scored_merge_diff_kernel(const float* __restrict__ partial, int n_splits, int n_heads, int group, int dv, T* __restrict__ out, int64_t ld_out,
                         float lambda, float eps, float gain) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, h = blockIdx.y, kv = h / group, j = h - kv * group;
  float o[4] = {0.f, 0.f, 0.f, 0.f};                    // (dv <= 512: four entries a thread at most)
  float sq = 0.f;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const int hm = (kv * 2 + m) * group + j;
    const float* src = partial + ((int64_t)row * 2 * n_heads + hm) * n_splits * (dv + 2);
    float mx = -INFINITY;
    for (int i = 0; i < n_splits; ++i) mx = fmaxf(mx, src[i * (dv + 2)]);
    float total = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float mi = src[i * (dv + 2)];
      if (mi != -INFINITY) total = fmaf(src[i * (dv + 2) + 1], expf(mi - mx), total);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int d = threadIdx.x + 128 * t;
      if (d < dv) {
        float y = 0.f;
        for (int i = 0; i < n_splits; ++i) {
          const float mi = src[i * (dv + 2)];
          if (mi != -INFINITY) y = fmaf(src[i * (dv + 2) + 2 + d], expf(mi - mx), y);
        }
        y /= total;
        o[t] = m == 0 ? y : fmaf(-lambda, y, o[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) sq = fmaf(o[t], o[t], sq);
  sq = block_sum(sq, scratch);
  const float f = gain / sqrtf(sq / (float)dv + eps);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int d = threadIdx.x + 128 * t;
    if (d < dv) out[(int64_t)row * ld_out + (int64_t)h * dv + d] = from_f32<T>(o[t] * f);
  }
}

template <typename T, int KPL, int DPL, int NW>
int launch_scored(const ScoredArgs& a, int n_seqs, int max_new, size_t smem, cudaStream_t stream) {
  constexpr int TR = RPW * NW, THREADS = 32 * NW;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(scored_attention_kernel<T, KPL, DPL, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "attention (scored): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  const int tok = TR / a.hp, group = a.n_heads / a.n_kv_heads, chunks = (group + a.hp - 1) / a.hp;
  dim3 grid(((max_new + tok - 1) / tok) * a.n_splits, n_seqs, a.n_kv_heads * chunks);
  kvad_launch(scored_attention_kernel<T, KPL, DPL, NW>, grid, dim3(THREADS), smem, stream, a);
  KVAD_CHECK_LAUNCH("attention_scored");
  if (a.n_splits > 1 && a.merge) {       // (rows are single tokens here: row = sequence)
    kvad_launch(scored_merge_kernel<T>, dim3(n_seqs, a.n_heads), dim3(a.dv <= 64 ? 64 : 128), 0, stream, (const float*)a.partial, a.n_splits,
                a.n_heads, a.dv, (T*)a.out, a.ld_out, (const T*)a.gate, a.ld_gate, a.out_f32);
    KVAD_CHECK_LAUNCH("attention_scored (merge)");
  }
  return KVAD_OK;
}

template <typename T>
int dispatch_scored(const ScoredArgs& a, int n_seqs, int max_new, cudaStream_t stream) {
  const size_t limit = 200 * 1024;
  const size_t dkp = (size_t)((a.dk + 3) & ~3);
  auto need = [&](int tk, int tr) {
    return ((size_t)tr * dkp + (size_t)tk * (dkp + 1) + (a.v_alias ? 0 : (size_t)tk * a.dv) + (size_t)tr * tk) * sizeof(float);
  };
  const int dpl = (a.dv + 31) / 32;
  // Long values make a block heavy in registers and shared memory, so that one block an SM is all that fits: prompts
  // then take blocks of eight warps (64 pairs against the same tile of keys) where those fit, single-token rows never.
  const bool wide = max_new > 1 && dpl >= 2 && need(64, 64) <= limit;
  const int kpl = need(64, 32) <= limit ? 2 : 1;
  const size_t smem = need(32 * kpl, wide ? 64 : 32);
  if (smem > limit) KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (scored): keys of %d and values of %d entries do not fit shared memory", a.dk, a.dv);
#define KVAD_SC(K, D, W) return launch_scored<T, K, D, W>(a, n_seqs, max_new, smem, stream)
#define KVAD_SC_D(K, W)                      \
  do {                                       \
    if (dpl <= 1) KVAD_SC(K, 1, W);          \
    if (dpl <= 2) KVAD_SC(K, 2, W);          \
    if (dpl <= 4) KVAD_SC(K, 4, W);          \
    if (dpl <= 8) KVAD_SC(K, 8, W);          \
    if (dpl <= 16) KVAD_SC(K, 16, W);        \
  } while (0)
  if (wide) {
    if (dpl <= 2) KVAD_SC(2, 2, 8);
    if (dpl <= 4) KVAD_SC(2, 4, 8);
    if (dpl <= 8) KVAD_SC(2, 8, 8);
    if (dpl <= 16) KVAD_SC(2, 16, 8);
  }
  if (kpl == 2) KVAD_SC_D(2, 4);
  else KVAD_SC_D(1, 4);
#undef KVAD_SC_D
#undef KVAD_SC
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (scored): values of %d entries are above this kernel's limit of 512", a.dv);
}

// Keys (dk a head) and values (dv a head) of a step's rows into their pages; with `v_other` the stored value is
// (1 - lambda) v + lambda v_other, lambda a scalar in device memory (32-bit arithmetic, one rounding).
template <typename T>
__global__ void kv_store_blend_kernel(const T* __restrict__ k_src, int64_t ld_k, const T* __restrict__ v_src, int64_t ld_v,
                                      const T* __restrict__ v_other, int64_t ld_o, const void* __restrict__ lambda, int lambda_f32,
                                      const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                      const int* __restrict__ page_table, int table_width, T* __restrict__ k_pages,
                                      T* __restrict__ v_pages, int n_rows, int n_kv, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int wk = n_kv * dk, wv = n_kv * dv, per_row = wk + wv;
  const float lam = v_other != nullptr ? load_param(lambda, 0, lambda_f32) : 0.f;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row), c = (int)(i % per_row);
    const int pos = row_pos[r];
    const int64_t page = page_table[(int64_t)row_seq[r] * table_width + pos / PAGE];
    if (c < wk) {
      const int h = c / dk, d = c % dk;
      k_pages[((page * n_kv + h) * PAGE + pos % PAGE) * dk + d] = k_src[(int64_t)r * ld_k + c];
    } else {
      const int cv = c - wk, h = cv / dv, d = cv % dv;
      T v = v_src[(int64_t)r * ld_v + cv];
      if (v_other != nullptr) v = from_f32<T>((1.0f - lam) * to_f32(v) + lam * to_f32(v_other[(int64_t)r * ld_o + cv]));
      v_pages[((page * n_kv + h) * PAGE + pos % PAGE) * dv + d] = v;
    }
  }
}

// Queries, keys and values of a step's rows, turned by the rows' positions where the layer asks for it, and the keys
// and values stored: the first `rot_k` entries of every query head are turned in place; every key head likewise on
// its way to its page; every value head over all its entries (`freq_v` given) or not at all.  A thread owns one unit
// of a row: a pair that turns, or one entry that passes.  Angles are position x frequency in 32-bit.
template <typename T>
__global__ void turn_store_kernel(T* __restrict__ q, int64_t ld_q, const T* __restrict__ k_src, int64_t ld_k, const T* __restrict__ v_src,
                                  int64_t ld_v, const float* __restrict__ freq_k, int rot_k, int inter_k,
                                  const float* __restrict__ freq_v, int inter_v, const int* __restrict__ row_seq,
                                  const int* __restrict__ row_pos, const int* __restrict__ page_table, int table_width,
                                  T* __restrict__ k_pages, T* __restrict__ v_pages, int n_rows, int n_heads, int n_kv, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int half_k = rot_k / 2, half_v = dv / 2;
  const int uq = n_heads * half_k;                         // queries: only the pairs that turn (the rest stay where they are)
  const int per_k = half_k + (dk - rot_k), uk = n_kv * per_k;
  const int per_v = freq_v != nullptr ? half_v : dv, uv = n_kv * per_v;
  const int per_row = uq + uk + uv;
  const int64_t total = (int64_t)n_rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row), c = (int)(i % per_row);
    const int pos = row_pos[r];
    if (c < uq) {
      const int h = c / half_k, p = c % half_k;
      const int a = inter_k ? 2 * p : p, b = inter_k ? 2 * p + 1 : p + half_k;
      T* x = q + (int64_t)r * ld_q + (int64_t)h * dk;
      float sn, cs;
      sincosf((float)pos * freq_k[p], &sn, &cs);
      const float u = to_f32(x[a]), v = to_f32(x[b]);
      x[a] = from_f32<T>(turn_first(u, v, cs, sn));
      x[b] = from_f32<T>(turn_second(u, v, cs, sn));
      continue;
    }
    const int64_t page = page_table[(int64_t)row_seq[r] * table_width + pos / PAGE];
    if (c < uq + uk) {
      const int ck = c - uq, h = ck / per_k, p = ck % per_k;
      const T* x = k_src + (int64_t)r * ld_k + (int64_t)h * dk;
      T* d = k_pages + ((page * n_kv + h) * PAGE + pos % PAGE) * dk;
      if (p < half_k) {
        const int a = inter_k ? 2 * p : p, b = inter_k ? 2 * p + 1 : p + half_k;
        float sn, cs;
        sincosf((float)pos * freq_k[p], &sn, &cs);
        const float u = to_f32(x[a]), v = to_f32(x[b]);
        d[a] = from_f32<T>(turn_first(u, v, cs, sn));
        d[b] = from_f32<T>(turn_second(u, v, cs, sn));
      } else {
        const int e = rot_k + (p - half_k);
        d[e] = x[e];
      }
    } else {
      const int cv = c - uq - uk, h = cv / per_v, p = cv % per_v;
      const T* x = v_src + (int64_t)r * ld_v + (int64_t)h * dv;
      T* d = v_pages + ((page * n_kv + h) * PAGE + pos % PAGE) * dv;
      if (freq_v != nullptr) {
        const int a = inter_v ? 2 * p : p, b = inter_v ? 2 * p + 1 : p + half_v;
        float sn, cs;
        sincosf((float)pos * freq_v[p], &sn, &cs);
        const float u = to_f32(x[a]), v = to_f32(x[b]);
        d[a] = from_f32<T>(turn_first(u, v, cs, sn));
        d[b] = from_f32<T>(turn_second(u, v, cs, sn));
      } else {
        d[p] = x[p];
      }
    }
  }
}

// Queries and keys RMS-normed in 32-bit (over `span` consecutive entries of their row at a time: one head, or the whole
// projection; a weight is as long as a span, absent weights are ones), then the first `rot` entries of every head turned by
// the row's position (pairs (i, i + rot/2); cosine and sine times `mscale`); queries are written back in place, keys
// go to their pages, values (n_v heads of dv) are stored as they are.  A block per row; the row's queries and keys
// lie in shared memory as 32-bit numbers while their sums of squares are taken, a warp per span.
template <typename T, bool VEC>
__global__ void __launch_bounds__(1024)
norm_turn_store_kernel(T* __restrict__ q, int64_t ld_q, const T* __restrict__ k_src, int64_t ld_k, const T* __restrict__ v_src, int64_t ld_v,
                       const void* __restrict__ wq, const void* __restrict__ wk, int w_f32, int span_q, int span_k,
                       float eps, const float* __restrict__ freq, int rot, float mscale, const int* __restrict__ row_seq,
                       const int* __restrict__ row_pos, const int* __restrict__ page_table, int table_width, T* __restrict__ k_pages,
                       T* __restrict__ v_pages, int n_heads, int n_kv, int n_v, int dk, int dv) {
  // VEC: rows are read and written in 16-byte pieces (head sizes, strides and addresses allow it); the arithmetic is the same
  constexpr int E = VEC ? 16 / (int)sizeof(T) : 1;
  extern __shared__ float nts[];
  const int nq = n_heads * dk, nk = n_kv * dk, spans_q = span_q > 0 ? nq / span_q : 0, spans_k = span_k > 0 ? nk / span_k : 0;
  float* xs = nts;                      // [nq + nk] the row's queries, then its keys
  float* inv = nts + nq + nk;           // [spans_q + spans_k]
  float* cs_t = inv + spans_q + spans_k;   // [rot / 2] cosines, then [rot / 2] sines: one per pair, shared by every head of the row
  float* sn_t = cs_t + rot / 2;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  const int pos = row_pos[r];
  const int64_t page = page_table[(int64_t)row_seq[r] * table_width + pos / PAGE];
  T* qr = q + (int64_t)r * ld_q;
  const T* kr = k_src + (int64_t)r * ld_k;
  const T* vr = v_src + (int64_t)r * ld_v;
  for (int i = tid; i < (nq + nk) / E; i += blockDim.x) {
    const int c = i * E;
    const T* src = c < nq ? qr + c : kr + (c - nq);
    if (VEC) {
      float f[E];
      unpack16(*reinterpret_cast<const uint4*>(src), f, T());
#pragma unroll
      for (int e = 0; e < E; ++e) xs[c + e] = f[e];
    } else {
      xs[c] = to_f32(*src);
    }
  }
  // (the values do not change: straight to their page, while the queries and keys are worked on)
  for (int i = tid; i < n_v * dv / E; i += blockDim.x) {
    const int c = i * E, h = c / dv, d = c - h * dv;
    T* dst = v_pages + ((page * n_v + h) * PAGE + pos % PAGE) * dv + d;
    if (VEC) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vr + c);
    else *dst = vr[c];
  }
  for (int p = tid; p < rot / 2; p += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * freq[p], &sn, &cs);
    cs_t[p] = cs * mscale;
    sn_t[p] = sn * mscale;
  }
  __syncthreads();
  const int half = rot / 2;
  const int hps_q = span_q > 0 ? span_q / dk : 1, hps_k = span_k > 0 ? span_k / dk : 1;       // heads that are normed together
  const bool by_head = hps_q == 1 && hps_k == 1;
  const float inv_dk = 1.0f / (float)dk;
  if (!by_head) {                                                  // several heads are normed together: their sums first, a warp per span
    for (int sp = warp; sp < spans_q + spans_k; sp += n_warps) {
      const bool is_q = sp < spans_q;
      const int len = is_q ? span_q : span_k;
      const float* x = is_q ? xs + sp * span_q : xs + nq + (sp - spans_q) * span_k;
      float sq = 0.f;
      for (int c = lane; c < len; c += 32) sq = fmaf(x[c], x[c], sq);
      sq = warp_sum(sq);
      if (lane == 0) inv[sp] = 1.0f / sqrtf(sq / (float)len + eps);
    }
    __syncthreads();
  }
  // A warp takes a head at a time, a lane an entry at a time: the entry is normed (a weight is as long as what is normed
  // together, so a head's entries find theirs at the head's place within its span), turned with its partner half the turned
  // entries away (read from shared memory, which nothing writes any more), and goes straight to the queries' row or the key's page.
  for (int hd = warp; hd < n_heads + n_kv; hd += n_warps) {
    const bool is_q = hd < n_heads;
    const int hl = is_q ? hd : hd - n_heads, span = is_q ? span_q : span_k, hps = is_q ? hps_q : hps_k;
    const float* x = xs + hd * dk;
    const int sp = hps == 1 ? hl : hl / hps;
    float f = 1.f;
    if (span > 0 && by_head) {
      float sq = 0.f;
      for (int e = lane; e < dk; e += 32) sq = fmaf(x[e], x[e], sq);
      f = rsqrtf(fmaf(warp_sum(sq), inv_dk, eps));
    } else if (span > 0) {
      f = inv[(is_q ? 0 : spans_q) + sp];
    }
    const void* w = span > 0 ? (is_q ? wq : wk) : nullptr;
    const int wbase = (hl - sp * hps) * dk;
    T* dst = is_q ? qr + hl * dk : k_pages + ((page * n_kv + hl) * PAGE + pos % PAGE) * dk;
    for (int e = lane; e < dk; e += 32) {
      float y = x[e] * f * (w ? load_param(w, wbase + e, w_f32) : 1.f);
      if (e < rot) {
        const int pe = e < half ? e + half : e - half, pr = e < half ? e : e - half;
        const float z = x[pe] * f * (w ? load_param(w, wbase + pe, w_f32) : 1.f);
        y = e < half ? turn_first(y, z, cs_t[pr], sn_t[pr]) : turn_second(z, y, cs_t[pr], sn_t[pr]);
      }
      dst[e] = from_f32<T>(y);
    }
  }
}

// Differential attention's last step.  `a` holds, per row, the maps' outputs in 32-bit, laid out [kv head][map][head of
// the group][dv]; head h = kv * group + j of the output gets o = a1 - lambda a2, over sqrt(mean(o^2) + eps), times `gain`.
// A warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ a, int64_t ld_a, T* __restrict__ out, int64_t ld_out, int n_rows, int n_heads, int group, int dv,
                    float lambda, float eps, float gain) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (int64_t)n_rows * n_heads) return;
  const int64_t row = item / n_heads;
  const int h = (int)(item % n_heads), kv = h / group, j = h - kv * group, lane = threadIdx.x & 31;
  const float* a1 = a + row * ld_a + ((int64_t)(kv * 2) * group + j) * dv;
  const float* a2 = a1 + (int64_t)group * dv;
  float sq = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float o = fmaf(-lambda, a2[d], a1[d]);
    sq = fmaf(o, o, sq);
  }
  sq = warp_sum(sq);
  const float f = gain / sqrtf(sq / (float)dv + eps);
  T* o_row = out + row * ld_out + (int64_t)h * dv;
  for (int d = lane; d < dv; d += 32) o_row[d] = from_f32<T>(fmaf(-lambda, a2[d], a1[d]) * f);
}

// A warp per row: the first `rank` entries are RMS-normalised with a weight, the last `rot` entries turned by
// the row's position (pairs interleaved or half apart), and the row goes to its place in pages of one head of
// rank + rot entries.
template <typename T>
__global__ void __launch_bounds__(128)
latent_store_kernel(const T* __restrict__ src, int64_t ld, const void* __restrict__ w, int w_f32, float eps,
                    const float* __restrict__ inv_freq, int interleaved, const int* __restrict__ row_seq,
                    const int* __restrict__ row_pos, const int* __restrict__ page_table, int table_width,
                    T* __restrict__ pages, int n_rows, int rank, int rot) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const T* x = src + (int64_t)r * ld;
  const int pos = row_pos[r];
  const int64_t page = page_table[(int64_t)row_seq[r] * table_width + pos / PAGE];
  T* dst = pages + (page * PAGE + pos % PAGE) * (rank + rot);
  float sq = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float v = to_f32(x[c]);
    sq = fmaf(v, v, sq);
  }
  sq = warp_sum(sq);
  const float inv = 1.0f / sqrtf(sq / (float)rank + eps);
  for (int c = lane; c < rank; c += 32) dst[c] = from_f32<T>(to_f32(x[c]) * inv * load_param(w, c, w_f32));
  const int half = rot / 2;
  for (int p = lane; p < half; p += 32) {
    const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
    float sn, cs;
    sincosf((float)pos * inv_freq[p], &sn, &cs);
    const float u = to_f32(x[rank + ia]), v = to_f32(x[rank + ib]);
    dst[rank + ia] = from_f32<T>(turn_first(u, v, cs, sn));
    dst[rank + ib] = from_f32<T>(turn_second(u, v, cs, sn));
  }
}

// Head-wise linear maps for a few rows: out[r, h, :] = W_h . a[r, h, :] with W [heads, n_out, n_in] - a latent
// road's queries carried into the latent's space, and its attended latents carried to values.  A block takes one
// head and 8 outputs (many small blocks: the maps are short chains of loads, and only blocks side by side hide
// them) and stages up to 8 rows' inputs of that head in shared memory (32-bit); a warp has 2 of the outputs and
// walks the inputs once for both, lanes striding, four trips' loads in flight; the sums meet by shuffles.
template <typename T>
__global__ void __launch_bounds__(128)
linear_heads_kernel(const T* __restrict__ a, int64_t ld_a, int head_stride_a, const T* __restrict__ w, T* __restrict__ out,
                    int64_t ld_out, int head_stride_out, int n_rows, int n_in, int n_out) {
  constexpr int MR = 8, OPW = 2;
  extern __shared__ float rows_in[];                  // [MR][n_in]
  pdl_launch_dependents();
  const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, o0 = blockIdx.y * (4 * OPW) + warp * OPW;
  const T* wh = w + (int64_t)h * n_out * n_in;
  pdl_wait();
  for (int r0 = 0; r0 < n_rows; r0 += MR) {
    const int nr = n_rows - r0 < MR ? n_rows - r0 : MR;
    __syncthreads();
#pragma unroll 4
    for (int i = threadIdx.x; i < MR * n_in; i += blockDim.x) {
      const int r = i / n_in, c = i - r * n_in;
      rows_in[i] = r < nr ? to_f32(a[(int64_t)(r0 + r) * ld_a + (int64_t)h * head_stride_a + c]) : 0.f;
    }
    __syncthreads();
    float acc[OPW][MR];
#pragma unroll
    for (int o = 0; o < OPW; ++o)
#pragma unroll
      for (int r = 0; r < MR; ++r) acc[o][r] = 0.f;
#pragma unroll 4
    for (int c = lane; c < n_in; c += 32) {
      float wv[OPW];
#pragma unroll
      for (int o = 0; o < OPW; ++o) wv[o] = o0 + o < n_out ? to_f32(wh[(int64_t)(o0 + o) * n_in + c]) : 0.f;
#pragma unroll
      for (int r = 0; r < MR; ++r) {
        const float x = rows_in[r * n_in + c];
#pragma unroll
        for (int o = 0; o < OPW; ++o) acc[o][r] = fmaf(wv[o], x, acc[o][r]);
      }
    }
#pragma unroll
    for (int o = 0; o < OPW; ++o)
#pragma unroll
      for (int r = 0; r < MR; ++r) {
        const float v = warp_sum(acc[o][r]);
        if (lane == 0 && r < nr && o0 + o < n_out) out[(int64_t)(r0 + r) * ld_out + (int64_t)h * head_stride_out + o0 + o] = from_f32<T>(v);
      }
  }
}

}  // namespace

KVAD_EXPORT int kvad_linear_heads(int dtype, const void* a, int64_t ld_a, int head_stride_a, const void* w, void* out, int64_t ld_out,
                                  int head_stride_out, int n_rows, int n_heads, int n_in, int n_out, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && n_in > 0 && n_out > 0, "linear_heads: bad sizes rows=%d heads=%d in=%d out=%d", n_rows, n_heads, n_in, n_out);
  KVAD_REQUIRE(n_heads <= 65535 * 32 && (n_out + 7) / 8 <= 65535, "linear_heads: %d heads x %d outputs are more than one launch takes", n_heads, n_out);
  const size_t smem = (size_t)8 * n_in * sizeof(float);
  if (smem > 48 * 1024) KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_heads: inputs of %d entries a head are above this kernel's limit of 1536", n_in);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_heads, (n_out + 7) / 8), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(linear_heads_kernel<float>, grid, block, smem, stream, (const float*)a, ld_a, head_stride_a, (const float*)w, (float*)out, ld_out,
                head_stride_out, n_rows, n_in, n_out);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(linear_heads_kernel<__nv_bfloat16>, grid, block, smem, stream, (const __nv_bfloat16*)a, ld_a, head_stride_a, (const __nv_bfloat16*)w,
                (__nv_bfloat16*)out, ld_out, head_stride_out, n_rows, n_in, n_out);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "linear_heads: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("linear_heads");
  return KVAD_OK;
}

// Rows of sequences packed one after another (`seq_starts`), each sequence's rows being its last positions
// (`kv_lens`: its length after the step).  `n_splits` > 1 (single-token rows only): the keys of a (row, head) are
// dealt out tile by tile to that many blocks, and a second kernel merges what they leave in `partial`
// (float32, rows x heads x n_splits x (dv + 2)).  `hp`: heads of a key/value group a block takes together (32 / hp
// tokens a block).  `v_pages` == `k_pages` and ld_v == ld_k: values are the keys' first dv entries.
KVAD_EXPORT int kvad_attention_scored(int dtype, const void* q, int64_t ld_q, void* out, int64_t ld_out, const void* gate,
                                      int64_t ld_gate, const int* seq_starts, const int* kv_lens, const int* page_table,
                                      int table_width, const void* k_pages, const void* v_pages, int n_seqs, int n_heads,
                                      int n_kv_heads, int dk, int dv, int page_size, int max_new, int hp, float scale,
                                      float softcap, float slope_span, int window, int keep_first, int n_splits, float* partial,
                                      int key_maps, int out_f32, int merge, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && n_heads > 0 && n_kv_heads > 0 && dk > 0 && dv > 0 && table_width > 0 && max_new >= 0,
               "attention (scored): bad sizes seqs=%d heads=%d kv_heads=%d dk=%d dv=%d", n_seqs, n_heads, n_kv_heads, dk, dv);
  KVAD_REQUIRE(n_heads % n_kv_heads == 0, "attention (scored): %d heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  KVAD_REQUIRE(hp >= 1 && hp <= 32, "attention (scored): %d heads a block (1..32)", hp);
  KVAD_REQUIRE(keep_first >= 0, "attention (scored): keep_first %d", keep_first);
  KVAD_REQUIRE(n_splits >= 1 && (n_splits == 1 || (max_new == 1 && partial != nullptr)),
               "attention (scored): keys are split over blocks for single-token rows only, and need room for the parts");
  if (page_size != PAGE)
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (scored): takes pages of %d positions, not %d", PAGE, page_size);
  KVAD_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, "attention (scored): %d sequences x %d heads are more than one launch takes", n_seqs, n_heads);
  if (n_seqs == 0 || max_new == 0) return KVAD_OK;
  const bool alias = v_pages == k_pages;
  KVAD_REQUIRE(key_maps >= 1 && n_kv_heads % key_maps == 0 && (key_maps == 1 || !alias), "attention (scored): %d key heads do not share values %d by %d", n_kv_heads, key_maps, key_maps);
  KVAD_REQUIRE(!out_f32 || gate == nullptr, "attention (scored): a 32-bit output takes no gate");
  KVAD_REQUIRE(!alias || dv <= dk, "attention (scored): values read from the keys cannot be longer than a key");
  ScoredArgs a;
  a.q = q; a.ld_q = ld_q; a.out = out; a.ld_out = ld_out; a.gate = gate; a.ld_gate = ld_gate;
  a.seq_starts = seq_starts; a.kv_lens = kv_lens; a.page_table = page_table; a.table_width = table_width;
  a.k_pages = k_pages; a.v_pages = v_pages;
  a.ld_k = dk; a.k_head_stride = (int64_t)PAGE * dk; a.k_page_stride = (int64_t)n_kv_heads * PAGE * dk;
  a.ld_v = alias ? dk : dv; a.v_head_stride = (int64_t)PAGE * a.ld_v; a.v_page_stride = (int64_t)(n_kv_heads / key_maps) * PAGE * a.ld_v;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.dk = dk; a.dv = dv; a.hp = hp; a.v_alias = alias ? 1 : 0;
  a.n_splits = n_splits; a.partial = partial; a.key_maps = key_maps; a.out_f32 = out_f32 ? 1 : 0; a.merge = merge ? 1 : 0;
  const int piece = dtype == KVAD_DTYPE_F32 ? 4 : 8;
  a.vec_k = (dk % piece == 0 && (reinterpret_cast<uintptr_t>(k_pages) & 15) == 0) ? 1 : 0;
  a.vec_v = (!alias && dv % piece == 0 && (reinterpret_cast<uintptr_t>(v_pages) & 15) == 0) ? 1 : 0;
  a.scale = scale; a.softcap = softcap; a.slope_span = slope_span; a.window = window; a.keep_first = window > 0 ? keep_first : 0;
  if (dtype == KVAD_DTYPE_F32) return dispatch_scored<float>(a, n_seqs, max_new, stream);
  if (dtype == KVAD_DTYPE_BF16) return dispatch_scored<__nv_bfloat16>(a, n_seqs, max_new, stream);
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "attention (scored): unknown dtype %d", dtype);
}

// rot_k: how many entries of a query/key head turn (0: none; even, at most dk); freq_v null: the values are stored as they are,
// else they turn over all dv entries (dv even).
KVAD_EXPORT int kvad_turn_store(int dtype, void* q, int64_t ld_q, const void* k_src, int64_t ld_k, const void* v_src, int64_t ld_v,
                                const float* freq_k, int rot_k, int inter_k, const float* freq_v, int inter_v, const int* row_seq,
                                const int* row_pos, const int* page_table, int table_width, void* k_pages, void* v_pages, int n_rows,
                                int n_heads, int n_kv, int dk, int dv, int page_size, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && n_kv > 0 && dk > 0 && dv > 0 && table_width > 0, "turn_store: bad sizes rows=%d heads=%d kv_heads=%d dk=%d dv=%d",
               n_rows, n_heads, n_kv, dk, dv);
  KVAD_REQUIRE(page_size == PAGE, "turn_store: pages of %d positions, not %d", PAGE, page_size);
  KVAD_REQUIRE(rot_k >= 0 && rot_k % 2 == 0 && rot_k <= dk && (rot_k == 0 || freq_k != nullptr), "turn_store: %d of %d key entries cannot turn in pairs", rot_k, dk);
  KVAD_REQUIRE(freq_v == nullptr || dv % 2 == 0, "turn_store: values of %d entries cannot turn in pairs", dv);
  KVAD_REQUIRE(q && k_src && v_src && k_pages && v_pages, "turn_store: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const int64_t per_row = (int64_t)n_heads * (rot_k / 2) + (int64_t)n_kv * (rot_k / 2 + dk - rot_k) + (int64_t)n_kv * (freq_v ? dv / 2 : dv);
  const int64_t total = (int64_t)n_rows * per_row;
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16)), block(threads);
#define KVAD_TS(T)                                                                                                                     \
  kvad_launch(turn_store_kernel<T>, grid, block, 0, stream, (T*)q, ld_q, (const T*)k_src, ld_k, (const T*)v_src, ld_v, freq_k, rot_k, inter_k, \
              freq_v, inter_v, row_seq, row_pos, page_table, table_width, (T*)k_pages, (T*)v_pages, n_rows, n_heads, n_kv, dk, dv)
  if (dtype == KVAD_DTYPE_F32) KVAD_TS(float);
  else if (dtype == KVAD_DTYPE_BF16) KVAD_TS(__nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "turn_store: unknown dtype %d", dtype);
#undef KVAD_TS
  KVAD_CHECK_LAUNCH("turn_store");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_kv_store_blend(int dtype, const void* k_src, int64_t ld_k, const void* v_src, int64_t ld_v, const void* v_other,
                                    int64_t ld_o, const void* lambda, int lambda_f32, const int* row_seq, const int* row_pos,
                                    const int* page_table, int table_width, void* k_pages, void* v_pages, int n_rows, int n_kv,
                                    int dk, int dv, int page_size, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_kv > 0 && dk > 0 && dv > 0 && table_width > 0, "kv_store_blend: bad sizes rows=%d kv_heads=%d dk=%d dv=%d", n_rows, n_kv, dk, dv);
  KVAD_REQUIRE(page_size == PAGE, "kv_store_blend: pages of %d positions, not %d", PAGE, page_size);
  KVAD_REQUIRE(v_other == nullptr || lambda != nullptr, "kv_store_blend: a blend needs its weight");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * n_kv * (dk + dv);
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16)), block(threads);
#define KVAD_ST(T)                                                                                                              \
  kvad_launch(kv_store_blend_kernel<T>, grid, block, 0, stream, (const T*)k_src, ld_k, (const T*)v_src, ld_v, (const T*)v_other, ld_o, \
              lambda, lambda_f32, row_seq, row_pos, page_table, table_width, (T*)k_pages, (T*)v_pages, n_rows, n_kv, dk, dv)
  if (dtype == KVAD_DTYPE_F32) KVAD_ST(float);
  else if (dtype == KVAD_DTYPE_BF16) KVAD_ST(__nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "kv_store_blend: unknown dtype %d", dtype);
#undef KVAD_ST
  KVAD_CHECK_LAUNCH("kv_store_blend");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_latent_store(int dtype, const void* src, int64_t ld, const void* w, int w_f32, float eps, const float* inv_freq,
                                  int interleaved, const int* row_seq, const int* row_pos, const int* page_table, int table_width,
                                  void* pages, int n_rows, int rank, int rot, int page_size, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && table_width > 0, "latent_store: bad sizes rows=%d rank=%d rot=%d", n_rows, rank, rot);
  KVAD_REQUIRE(page_size == PAGE, "latent_store: pages of %d positions, not %d", PAGE, page_size);
  KVAD_REQUIRE(w != nullptr && (rot == 0 || inv_freq != nullptr), "latent_store: needs the norm's weight and the frequencies");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid((n_rows + 3) / 4), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(latent_store_kernel<float>, grid, block, 0, stream, (const float*)src, ld, w, w_f32, eps, inv_freq, interleaved, row_seq,
                row_pos, page_table, table_width, (float*)pages, n_rows, rank, rot);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(latent_store_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)src, ld, w, w_f32, eps, inv_freq,
                interleaved, row_seq, row_pos, page_table, table_width, (__nv_bfloat16*)pages, n_rows, rank, rot);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "latent_store: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("latent_store");
  return KVAD_OK;
}

// span_q / span_k: how many consecutive entries of the queries' / keys' projection are normed together (0: no norm; a
// multiple of dk that divides the projection); wq / wk: the norms' weights (as long as what is normed together, float32 or
// bfloat16; null: ones).  n_v: value heads (the pages of values have that many).  rot: entries of a head that turn (even, at most dk).
KVAD_EXPORT int kvad_norm_turn_store(int dtype, void* q, int64_t ld_q, const void* k_src, int64_t ld_k, const void* v_src, int64_t ld_v,
                                     const void* wq, const void* wk, int w_f32, int span_q, int span_k, float eps,
                                     const float* freq, int rot, float mscale, const int* row_seq, const int* row_pos, const int* page_table,
                                     int table_width, void* k_pages, void* v_pages, int n_rows, int n_heads, int n_kv, int n_v, int dk, int dv,
                                     int page_size, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && n_kv > 0 && n_v > 0 && dk > 0 && dv > 0 && table_width > 0,
               "norm_turn_store: bad sizes rows=%d heads=%d kv_heads=%d value heads=%d dk=%d dv=%d", n_rows, n_heads, n_kv, n_v, dk, dv);
  KVAD_REQUIRE(page_size == PAGE, "norm_turn_store: pages of %d positions, not %d", PAGE, page_size);
  KVAD_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk && (rot == 0 || freq != nullptr), "norm_turn_store: %d of %d key entries cannot turn in pairs", rot, dk);
  KVAD_REQUIRE(span_q >= 0 && span_k >= 0 && (span_q == 0 || (span_q % dk == 0 && (n_heads * dk) % span_q == 0)) &&
               (span_k == 0 || (span_k % dk == 0 && (n_kv * dk) % span_k == 0)), "norm_turn_store: norms over %d and %d entries do not fit heads of %d", span_q, span_k, dk);
  KVAD_REQUIRE((wq == nullptr || span_q > 0) && (wk == nullptr || span_k > 0), "norm_turn_store: a weight goes with a norm");
  KVAD_REQUIRE(q && k_src && v_src && k_pages && v_pages, "norm_turn_store: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const int nq = n_heads * dk, nk = n_kv * dk;
  const size_t smem = ((size_t)nq + nk + (span_q ? nq / span_q : 0) + (span_k ? nk / span_k : 0) + rot) * sizeof(float);
  KVAD_REQUIRE(smem <= 200 * 1024, "norm_turn_store: rows of %d queries and keys do not fit shared memory", nq + nk);
  // many rows: short rows take smaller blocks, more rows an SM; few rows (single tokens): a warp per head, so that no warp walks several
  const int per_head = 32 * (n_heads + n_kv);
  const int threads = n_rows <= 2 * 148 ? (per_head > 1024 ? 1024 : (per_head < 128 ? 128 : per_head)) : (nq + nk >= 2048 ? 256 : 128);
#define KVAD_NTS(T)                                                                                                                          \
  do {                                                                                                                                       \
    static size_t configured = 0;                                                                                                            \
    if (smem > 48 * 1024 && smem > configured) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(norm_turn_store_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (e == cudaSuccess) e = cudaFuncSetAttribute(norm_turn_store_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "norm_turn_store: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                                                     \
    }                                                                                                                                        \
    const int piece = 16 / (int)sizeof(T);                                                                                                   \
    const bool vec = dk % piece == 0 && dv % piece == 0 && ld_q % piece == 0 && ld_k % piece == 0 && ld_v % piece == 0 &&                    \
                     ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_src) | reinterpret_cast<uintptr_t>(v_src) |            \
                       reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0;                              \
    if (vec)                                                                                                                                 \
      kvad_launch(norm_turn_store_kernel<T, true>, dim3(n_rows), dim3(threads), smem, stream, (T*)q, ld_q, (const T*)k_src, ld_k, (const T*)v_src, ld_v, \
                  wq, wk, w_f32, span_q, span_k, eps, freq, rot, mscale, row_seq, row_pos, page_table, table_width,          \
                  (T*)k_pages, (T*)v_pages, n_heads, n_kv, n_v, dk, dv);                                                                     \
    else                                                                                                                                     \
      kvad_launch(norm_turn_store_kernel<T, false>, dim3(n_rows), dim3(threads), smem, stream, (T*)q, ld_q, (const T*)k_src, ld_k, (const T*)v_src, ld_v, \
                  wq, wk, w_f32, span_q, span_k, eps, freq, rot, mscale, row_seq, row_pos, page_table, table_width,          \
                  (T*)k_pages, (T*)v_pages, n_heads, n_kv, n_v, dk, dv);                                                                     \
  } while (0)
  if (dtype == KVAD_DTYPE_F32) KVAD_NTS(float);
  else if (dtype == KVAD_DTYPE_BF16) KVAD_NTS(__nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "norm_turn_store: unknown dtype %d", dtype);
#undef KVAD_NTS
  KVAD_CHECK_LAUNCH("norm_turn_store");
  return KVAD_OK;
}

// partial: what kvad_attention_scored left with `merge` 0 for 2 x n_heads query heads ([kv head][map][head of the group]) of
// single-token rows; out: [rows, n_heads x dv] of `dtype`.
KVAD_EXPORT int kvad_scored_merge_diff(int dtype, const float* partial, int n_splits, int n_rows, int n_heads, int group, int dv, void* out,
                                       int64_t ld_out, float lambda, float eps, float gain, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_splits >= 1 && n_heads > 0 && group > 0 && n_heads % group == 0 && dv > 0 && dv <= 512 && partial && out,
               "scored_merge_diff: bad arguments");
  KVAD_REQUIRE(n_rows <= 2147483647 && n_heads <= 65535, "scored_merge_diff: too many heads for one launch");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows, n_heads), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(scored_merge_diff_kernel<float>, grid, block, 0, stream, partial, n_splits, n_heads, group, dv, (float*)out, ld_out, lambda, eps, gain);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(scored_merge_diff_kernel<__nv_bfloat16>, grid, block, 0, stream, partial, n_splits, n_heads, group, dv, (__nv_bfloat16*)out, ld_out,
                lambda, eps, gain);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "scored_merge_diff: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("scored_merge_diff");
  return KVAD_OK;
}

// a: float32 [rows, 2 heads x dv] as the attention left it ([kv head][map][head of the group][dv]); out: [rows, heads x dv].
KVAD_EXPORT int kvad_diff_combine(int dtype, const float* a, int64_t ld_a, void* out, int64_t ld_out, int n_rows, int n_heads, int group, int dv,
                                  float lambda, float eps, float gain, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && group > 0 && n_heads % group == 0 && dv > 0 && a && out, "diff_combine: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const int64_t items = (int64_t)n_rows * n_heads;
  dim3 grid((unsigned)((items + 3) / 4)), block(128);
  if (dtype == KVAD_DTYPE_F32) kvad_launch(diff_combine_kernel<float>, grid, block, 0, stream, a, ld_a, (float*)out, ld_out, n_rows, n_heads, group, dv, lambda, eps, gain);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(diff_combine_kernel<__nv_bfloat16>, grid, block, 0, stream, a, ld_a, (__nv_bfloat16*)out, ld_out, n_rows, n_heads, group, dv, lambda, eps, gain);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "diff_combine: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("diff_combine");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
