// Softmax attention whose scores are capped, whose keys and values have different widths, and
// whose q, k and v pass a short causal filter over time before the rotation.  Plain kernels for
// any precision and size; the arithmetic for one (token, head) depends on its position and the
// cache alone, so prompts, parts of prompts and single tokens give the same bits.
//
//   gb_filter_rope_cache:  u [T, q | k | v] -> filter over time -> RMS norm of every q and k head
//                          with a weight over its dims (when weights are given) -> rotation of the
//                          first `rot` dims of every q and k head (dim i pairs with i + rot/2; angle
//                          float(pos) * inv_freq[i], float32; cosines and sines times `rot_mag`) ->
//                          q times 1 + qt_coef ln(floor((pos + 1) / qt_every) + 1) (when qt_every)
//                          -> q rows, keys and values into pages.  With `v_from_k` the rows hold
//                          q | k only and a value head is its key head as projected and filtered,
//                          before norm and rotation
//   gb_attention_capped:   score = (q . k) * scale; score <- cap * tanh(score / cap) when cap > 0;
//                          keys lo..p with lo = max(0, p + 1 - window), and with `keep_first` the
//                          keys 0..keep_first-1 as well, wherever the window stands; softmax, whose
//                          denominator also holds exp(sink[head]) when sinks are given (a term
//                          without key or value); output times sigmoid(gate) * out_scale when a
//                          gate is given
//
// Cache layout as everywhere in the package: keys [pages, kv_heads, page_size, D], values
// transposed inside a page [pages, kv_heads, Vd, page_size].
#include "common.cuh"

constexpr int CHUNK = 128;
constexpr int MAX_TAPS = 8;
constexpr int VPT = 4;   // value dims a thread keeps: values up to VPT * CHUNK wide

template <typename T>
__device__ __forceinline__ float filtered(const T* __restrict__ u, long long ldu, int row0, int local,
                                          const float* __restrict__ hist, const float* __restrict__ taps, int C, int c, int K) {
  float acc = 0.f;
  for (int j = 0; j < K; ++j) {
    const int at = local - (K - 1) + j;
    const float in = at >= 0 ? to_f32(u[(size_t)(row0 + at) * ldu + c]) : hist[(size_t)(K - 1 + at) * C + c];
    acc = fmaf(taps[(size_t)c * K + j], in, acc);
  }
  return acc;
}

// One block per (token, head): the H query heads, then the G key heads, then the G value heads.
// A q or k head is filtered into shared memory first, a dim a thread, beside the cosines and sines
// of the token's angles; then every dim takes its partner from there (with each thread filtering
// its partner again and taking its own sine and cosine, the kernel was bound by instructions).
constexpr int MAX_HEAD = 512;

template <typename T>
__global__ void __launch_bounds__(128) filter_rope_cache_kernel(
    const T* __restrict__ u, long long ldu, const float* __restrict__ taps, const float* __restrict__ state, int K,
    const float* __restrict__ inv_freq, int rot, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
    const int* __restrict__ seq_slot, const int* __restrict__ cu, const int* __restrict__ page_table, int table_width,
    int page_size, T* __restrict__ q_out, long long ldq, T* __restrict__ kcache, T* __restrict__ vcache, int H, int G, int D,
    int Vd, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float norm_eps, float rot_mag, float qt_coef,
    int qt_every, int v_from_k) {
  __shared__ float vals[MAX_HEAD], cs[MAX_HEAD];   // cs: cos[rot / 2], then sin[rot / 2]
  __shared__ float scratch[33];
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, hh = blockIdx.y, b = tok_seq[t], pos = tok_pos[t], slot = seq_slot[b];
  const int row0 = cu[b], local = t - row0, half = rot / 2;
  const int C = (H + G) * D + (v_from_k ? 0 : G * Vd);
  const float* hist = K > 1 ? state + (size_t)slot * (K - 1) * C : nullptr;
  const int page = page_table ? page_table[(size_t)slot * table_width + (pos / page_size) % table_width] : 0;
  const int off = pos % page_size;
  if (hh >= H + G) {                  // a value head: filtered, then into its page (a dim's positions contiguous)
    if (!vcache) return;
    const int g = hh - H - G;
    for (int d = threadIdx.x; d < Vd; d += blockDim.x) {
      const int c = (v_from_k ? H * D : (H + G) * D) + g * Vd + d;
      const float val = K > 1 ? filtered(u, ldu, row0, local, hist, taps, C, c, K) : to_f32(u[(size_t)t * ldu + c]) * (K == 1 ? taps[c] : 1.f);
      vcache[(((size_t)page * G + g) * Vd + d) * page_size + off] = from_f32<T>(val);
    }
    return;
  }
  if (hh >= H && !kcache) return;
  const float* norm_w = hh < H ? q_norm : k_norm;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const int e = hh * D + i;
    const float x = K > 1 ? filtered(u, ldu, row0, local, hist, taps, C, e, K) : to_f32(u[(size_t)t * ldu + e]) * (K == 1 ? taps[e] : 1.f);
    vals[i] = x;
    ss = fmaf(x, x, ss);
    if (i < half) {
      float sn, cn;
      sincosf((float)pos * inv_freq[i], &sn, &cn);
      cs[half + i] = sn * rot_mag;
      cs[i] = cn * rot_mag;
    }
  }
  if (norm_w) {            // the head divided by its root mean square, times the weight of each dim
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)D + norm_eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) vals[i] = vals[i] * inv * norm_w[i];
  }
  __syncthreads();
  const float temper = (hh < H && qt_every > 0) ? 1.0f + qt_coef * logf((float)((pos + 1) / qt_every + 1)) : 1.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float val = vals[i];
    if (i < rot) {
      // the pair (a, b) = (dim j, dim j + half) becomes (a cos - b sin, b cos + a sin)
      const int j = i < half ? i : i - half;
      val = i < half ? val * cs[j] - vals[i + half] * cs[half + j] : val * cs[j] + vals[i - half] * cs[half + j];
    }
    if (hh < H) q_out[(size_t)t * ldq + hh * D + i] = from_f32<T>(val * temper);
    else kcache[(((size_t)page * G + (hh - H)) * page_size + off) * D + i] = from_f32<T>(val);
  }
}

// taps: [(H + G) D + G Vd, K] float32 (K = 0: no filter); state: [slots, K - 1, channels] float32.
// G = 0: the rows hold queries only (a layer that reads another layer's keys and values).
// q_norm, k_norm: float32 [D] or null; v_from_k needs Vd == D.
GB_EXPORT int gb_filter_rope_cache_ext(const void* u, int dtype, long long ldu, const float* taps, const float* state, int K,
                                       const float* inv_freq, int rot, const int* tok_pos, const int* tok_seq,
                                       const int* seq_slot, const int* cu, const int* page_table, int table_width,
                                       int page_size, void* q_out, long long ldq, void* kcache, void* vcache, int ntok, int H,
                                       int G, int D, int Vd, const float* q_norm, const float* k_norm, float norm_eps,
                                       float rot_mag, float qt_coef, int qt_every, int v_from_k, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (K < 0 || K > MAX_TAPS || rot < 0 || rot > D || rot % 2 || H <= 0 || G < 0 || D <= 0 || D > MAX_HEAD || Vd <= 0)
    return GB_ERR_SIZE;
  if (v_from_k && (Vd != D || K > 1)) return GB_ERR_SIZE;
  if ((K > 0 && !taps) || (K > 1 && !state) || (rot > 0 && !inv_freq) || qt_every < 0) return GB_ERR_ARG;
  const dim3 grid(ntok, H + 2 * G);
  if (dtype == GB_F32)
    gb_launch(filter_rope_cache_kernel<float>, grid, 128, 0, stream, (const float*)u, ldu, taps, state, K, inv_freq, rot,
              tok_pos, tok_seq, seq_slot, cu, page_table, table_width, page_size, (float*)q_out, ldq, (float*)kcache,
              (float*)vcache, H, G, D, Vd, q_norm, k_norm, norm_eps, rot_mag, qt_coef, qt_every, v_from_k);
  else if (dtype == GB_BF16)
    gb_launch(filter_rope_cache_kernel<bf16>, grid, 128, 0, stream, (const bf16*)u, ldu, taps, state, K, inv_freq, rot,
              tok_pos, tok_seq, seq_slot, cu, page_table, table_width, page_size, (bf16*)q_out, ldq, (bf16*)kcache,
              (bf16*)vcache, H, G, D, Vd, q_norm, k_norm, norm_eps, rot_mag, qt_coef, qt_every, v_from_k);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

GB_EXPORT int gb_filter_rope_cache(const void* u, int dtype, long long ldu, const float* taps, const float* state, int K,
                                   const float* inv_freq, int rot, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                   const int* cu, const int* page_table, int table_width, int page_size, void* q_out,
                                   long long ldq, void* kcache, void* vcache, int ntok, int H, int G, int D, int Vd,
                                   cudaStream_t stream) {
  return gb_filter_rope_cache_ext(u, dtype, ldu, taps, state, K, inv_freq, rot, tok_pos, tok_seq, seq_slot, cu, page_table,
                                  table_width, page_size, q_out, ldq, kcache, vcache, ntok, H, G, D, Vd, nullptr, nullptr, 0.f,
                                  1.f, 0.f, 0, 0, stream);
}

// One block per (token, query head); online softmax over chunks of 128 keys: first the kept keys
// below the window (chunks from 0), then the window (chunks from lo).  A sink starts the running
// maximum at its value and the running sum at one.
template <typename T>
__global__ void __launch_bounds__(CHUNK) attention_capped_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride, const T* __restrict__ kcache,
    const T* __restrict__ vcache, const int* __restrict__ page_table, int table_width, int page_size, int G, int D, int Vd,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, int H, int window,
    int keep_first, const float* __restrict__ sink, float scale, float cap, const T* __restrict__ gate, long long gate_stride,
    float out_scale) {
  extern __shared__ float smem[];
  pdl_release_next();
  pdl_wait_prior();
  float* qs = smem;                    // [D]
  float* p = qs + D;                   // [CHUNK]
  float* scratch = p + CHUNK;          // [34]
  size_t* rows = (size_t*)(((uintptr_t)(scratch + 34) + 7) & ~(uintptr_t)7);   // [CHUNK]
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (H / G);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int hi = pos + 1;
  const int lo = window > 0 ? max(0, hi - window) : 0;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * D;
  for (int i = tid; i < D; i += CHUNK) qs[i] = to_f32(qrow[i]);
  __syncthreads();
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f, acc[VPT] = {};
  const int kept = min(keep_first, lo);          // kept keys that the window does not cover
  const int kept_chunks = (kept + CHUNK - 1) / CHUNK;
  for (int it = 0; it < kept_chunks || lo + (it - kept_chunks) * CHUNK < hi; ++it) {
    const int c0 = it < kept_chunks ? it * CHUNK : lo + (it - kept_chunks) * CHUNK;
    const int end = it < kept_chunks ? kept : hi;
    const int j = c0 + tid;
    float s = -INFINITY;
    if (j < end) {
      const int page = page_table[(size_t)slot * table_width + (j / page_size) % table_width];
      const int off = j % page_size;
      const T* kr = kcache + (((size_t)page * G + g) * page_size + off) * D;
      rows[tid] = ((size_t)page * G + g) * Vd * page_size + off;
      float d = 0.f;
      for (int i = 0; i < D; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
      s = d * scale;
      if (cap > 0.f) s = cap * tanhf(s * inv_cap);
    }
    const float m_new = fmaxf(m, block_max(s, scratch));
    const float pj = j < end ? expf(s - m_new) : 0.f;
    p[tid] = pj;
    const float csum = block_sum(pj, scratch);   // also orders the writes of p and rows
    const float alpha = expf(m - m_new);
    l = l * alpha + csum;
    const int n = min(CHUNK, end - c0);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int d = tid + u * CHUNK;
      if (d < Vd) {
        float a = acc[u] * alpha;
        for (int jj = 0; jj < n; ++jj) a = fmaf(p[jj], to_f32(vcache[rows[jj] + (size_t)d * page_size]), a);
        acc[u] = a;
      }
    }
    m = m_new;
    __syncthreads();
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * Vd;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int d = tid + u * CHUNK;
    if (d < Vd) {
      float o = acc[u] / l;
      if (gate) o *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + (size_t)h * Vd + d])));
      orow[d] = from_f32<T>(o * out_scale);
    }
  }
}

GB_EXPORT int gb_attention_capped(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                  const void* kcache, const void* vcache, const int* page_table, int table_width, int page_size,
                                  int G, int D, int Vd, const int* tok_pos, const int* tok_seq, const int* seq_slot, int ntok,
                                  int H, int window, int keep_first, const float* sink, float scale, float cap,
                                  const void* gate, long long gate_stride, float out_scale, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (D <= 0 || Vd <= 0 || Vd > VPT * CHUNK || G <= 0 || H % G || keep_first < 0) return GB_ERR_SIZE;
  if (window <= 0) keep_first = 0;      // every key is seen already
  const size_t smem = (size_t)(D + CHUNK + 34) * sizeof(float) + CHUNK * sizeof(size_t) + 8;
  dim3 grid(ntok, H);
  if (dtype == GB_F32)
    gb_launch(attention_capped_kernel<float>, grid, CHUNK, smem, stream, (const float*)q, q_stride, (float*)out, out_stride,
              (const float*)kcache, (const float*)vcache, page_table, table_width, page_size, G, D, Vd, tok_pos, tok_seq,
              seq_slot, H, window, keep_first, sink, scale, cap, (const float*)gate, gate_stride, out_scale);
  else if (dtype == GB_BF16)
    gb_launch(attention_capped_kernel<bf16>, grid, CHUNK, smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,
              (const bf16*)kcache, (const bf16*)vcache, page_table, table_width, page_size, G, D, Vd, tok_pos, tok_seq, seq_slot,
              H, window, keep_first, sink, scale, cap, (const bf16*)gate, gate_stride, out_scale);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}
