// Routed feed-forward (mixture of experts): the router and the token-major expert kernels.
//
//   z[t, e]  = router[e] . h[t] + bias[e]                       (float32)
//   chosen   = the `top` largest z (the lower index wins a tie); weight = softmax over the chosen z
//   expert:    g = min(gate h, limit), u = clamp(up h, -limit, limit)
//              y = g * sigmoid(alpha g) * (u + shift);  out = down y
//   residual[t] += sum over chosen of weight * expert_e(h[t])  +  sigmoid(sg . h[t]) * shared(h[t])
//
// Two more forms for designs that ask for them: `all_softmax` (the weights are the chosen experts'
// shares of the softmax over ALL experts, not renormalized), and experts without a gate
// (gb_moe_up: y = gelu(up h) with the exact, erf form; out = down y; the first matrices are [E, ff, width]).
//
// The router's logits are a product like any other (the part computes them in float32); this unit
// picks the experts from them and runs the experts token-major: a block owns one (token, chosen
// expert) pair and a run of the expert's features, so the kernels need nothing from the host about
// who chose what and run inside captured steps.  Every pair's down product leaves a weighted
// float32 row, and a token's rows are added into the residual in the order of its chosen list,
// then the shared expert: the same bits whatever else is in the batch.  All sums are float32.
#include "common.cuh"

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; typedef float4 type; };
template <> struct Vec<bf16> { static constexpr int N = 8; typedef uint4 type; };

__device__ __forceinline__ void unpack(const float4& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
__device__ __forceinline__ void unpack(const uint4& v, float* f) {
  const __nv_bfloat162* p = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(p[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

// Lanes' shares of two rows . xs (xs float32 in shared memory) at once, so that twice the loads are
// in flight; the caller adds the lanes with warp_sum.  `vec`: the rows start on 16-byte boundaries
// and n is a multiple of the vector width.
template <typename T>
__device__ __forceinline__ void lane_dot2(const T* __restrict__ r0, const T* __restrict__ r1, const float* __restrict__ xs,
                                          int n, int lane, bool vec, float& a0, float& a1) {
  a0 = a1 = 0.f;
  if (vec) {
    constexpr int V = Vec<T>::N;
    const typename Vec<T>::type* p0 = (const typename Vec<T>::type*)r0;
    const typename Vec<T>::type* p1 = (const typename Vec<T>::type*)r1;
#pragma unroll 2
    for (int i = lane; i < n / V; i += 32) {
      float f0[V], f1[V];
      const typename Vec<T>::type v0 = p0[i], v1 = p1[i];
      unpack(v0, f0);
      unpack(v1, f1);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float x = xs[i * V + k];
        a0 = fmaf(f0[k], x, a0);
        a1 = fmaf(f1[k], x, a1);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) {
      a0 = fmaf(to_f32(r0[i]), xs[i], a0);
      a1 = fmaf(to_f32(r1[i]), xs[i], a1);
    }
  }
}

template <typename T> __device__ __forceinline__ bool rows_vectorize(const T* base, int n) {
  return n % Vec<T>::N == 0 && ((uintptr_t)base & 15) == 0;
}

// ---- router: the logits come from a product (float32 [ntok, ldz]); a warp per token adds the
// bias, picks the `top` largest (the lower index wins a tie) and takes the softmax over those
// alone.  Column E of z, when there is one, is the shared expert's gate logit.
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ zin, long long ldz,
                                                       const float* __restrict__ bias, int* __restrict__ idx,
                                                       float* __restrict__ wts, float* __restrict__ sg, int ntok, int E,
                                                       int top, int has_gate, int all_softmax) {
  extern __shared__ float smem[];
  pdl_release_next();
  pdl_wait_prior();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= ntok) return;
  float* z = smem + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) z[e] = zin[(size_t)t * ldz + e] + (bias ? bias[e] : 0.f);
  if (has_gate && lane == 0) sg[t] = 1.0f / (1.0f + expf(-zin[(size_t)t * ldz + E]));
  __syncwarp();
  float mine = 0.f, first = 0.f;   // lane k keeps the k-th chosen logit
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (k == 0) first = best;
    if (lane == k) mine = best;
    if (lane == 0) {
      idx[(size_t)t * top + k] = at < E ? at : 0;
      if (at < E) z[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float e = lane < top ? expf(mine - first) : 0.f;
  float sum = warp_sum(e);
  if (all_softmax) {               // the experts not chosen join the denominator (the chosen ones' places hold -inf: nothing)
    float rest = 0.f;
    for (int i = lane; i < E; i += 32) rest += expf(z[i] - first);
    sum += warp_sum(rest);
  }
  if (lane < top) wts[(size_t)t * top + lane] = e / sum;
}

// ---- gate and up of one (token, slot): FEATS features a block, a warp per feature in turn
constexpr int FEATS = 32;

template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, long long ldh,
                                                          const int* __restrict__ idx, const T* __restrict__ w_gu,
                                                          const T* __restrict__ ws_gu, T* __restrict__ y, int width,
                                                          int ff, int ffs, int ffmax, int top, int slots, float limit,
                                                          float limit_s, float alpha, float shift) {
  extern __shared__ float xs[];   // [width]
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x / slots, s = blockIdx.x % slots;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool routed = s < top;
  const int nf = routed ? ff : ffs;
  const int f0 = blockIdx.y * FEATS;
  if (f0 >= nf) return;
  const T* W = routed ? w_gu + (size_t)idx[(size_t)t * top + s] * 2 * ff * width : ws_gu;
  const float lim = routed ? limit : limit_s;
  for (int i = tid; i < width; i += 256) xs[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const bool vec = rows_vectorize(W, width);
  for (int f = f0 + warp; f < min(nf, f0 + FEATS); f += 8) {
    float g, u;
    lane_dot2(W + (size_t)f * width, W + (size_t)(nf + f) * width, xs, width, lane, vec, g, u);
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
      g = fminf(g, lim);
      u = fminf(fmaxf(u, -lim), lim);
      const float a = g / (1.0f + expf(-alpha * g)) * (u + shift);
      y[((size_t)t * slots + s) * ffmax + f] = from_f32<T>(a);
    }
  }
}

// ---- the same for experts without a gate: y = gelu(up h) (erf form), two features a warp at a time
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

template <typename T>
__global__ void __launch_bounds__(256) moe_up_kernel(const T* __restrict__ h, long long ldh, const int* __restrict__ idx,
                                                     const T* __restrict__ w_up, T* __restrict__ y, int width, int ff, int top) {
  extern __shared__ float xs[];   // [width]
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x / top, s = blockIdx.x % top;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int f0 = blockIdx.y * FEATS;
  if (f0 >= ff) return;
  const T* W = w_up + (size_t)idx[(size_t)t * top + s] * ff * width;
  for (int i = tid; i < width; i += 256) xs[i] = to_f32(h[(size_t)t * ldh + i]);
  __syncthreads();
  const bool vec = rows_vectorize(W, width);
  for (int f = f0 + warp * 2; f < min(ff, f0 + FEATS); f += 16) {
    float a, b;
    const bool two = f + 1 < ff;
    lane_dot2(W + (size_t)f * width, W + (size_t)(two ? f + 1 : f) * width, xs, width, lane, vec, a, b);
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
      y[((size_t)t * top + s) * ff + f] = from_f32<T>(gelu_erf_f(a));
      if (two) y[((size_t)t * top + s) * ff + f + 1] = from_f32<T>(gelu_erf_f(b));
    }
  }
}

// ---- down of one (token, slot), weighted, into a float32 row of its own; the rows of a token are
// added into the residual in slot order by moe_sum_kernel
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T* __restrict__ y, const int* __restrict__ idx,
                                                       const float* __restrict__ wts, const float* __restrict__ sg,
                                                       const T* __restrict__ w_d, const T* __restrict__ ws_d,
                                                       float* __restrict__ rows, int width, int ff, int ffs, int ffmax,
                                                       int top, int slots) {
  extern __shared__ float ys[];   // [ffmax]
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x / slots, s = blockIdx.x % slots;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool routed = s < top;
  const int nf = routed ? ff : ffs;
  for (int i = tid; i < nf; i += 256) ys[i] = to_f32(y[((size_t)t * slots + s) * ffmax + i]);
  __syncthreads();
  const T* W = routed ? w_d + (size_t)idx[(size_t)t * top + s] * width * ff : ws_d;
  const float wt = routed ? wts[(size_t)t * top + s] : sg[t];
  const bool vec = rows_vectorize(W, nf);
  const int n0 = blockIdx.y * FEATS;
  for (int n = n0 + warp * 2; n < min(width, n0 + FEATS); n += 16) {
    float a, b;
    const bool two = n + 1 < width;
    lane_dot2(W + (size_t)n * nf, W + (size_t)(two ? n + 1 : n) * nf, ys, nf, lane, vec, a, b);
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
      rows[((size_t)t * slots + s) * width + n] = a * wt;
      if (two) rows[((size_t)t * slots + s) * width + n + 1] = b * wt;
    }
  }
}

__global__ void __launch_bounds__(256) moe_sum_kernel(const float* __restrict__ rows, float* __restrict__ residual,
                                                      long long ldr, int width, int slots) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  for (int n = blockIdx.y * 256 + threadIdx.x; n < width; n += gridDim.y * 256) {
    float total = 0.f;
    for (int s = 0; s < slots; ++s) total += rows[((size_t)t * slots + s) * width + n];
    residual[(size_t)t * ldr + n] += total;
  }
}

GB_EXPORT int gb_moe_topk_mode(const float* z, long long ldz, const float* bias, int* idx, float* wts, float* sg, int ntok,
                               int E, int top, int has_gate, int all_softmax, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (E <= 0 || top <= 0 || top > 32 || top > E || E > 2048) return GB_ERR_SIZE;
  gb_launch(moe_topk_kernel, dim3((ntok + 3) / 4), dim3(128), (size_t)4 * E * sizeof(float), stream, z, ldz, bias, idx, wts, sg,
            ntok, E, top, has_gate, all_softmax);
  return gb_launch_status();
}

GB_EXPORT int gb_moe_topk(const float* z, long long ldz, const float* bias, int* idx, float* wts, float* sg, int ntok,
                          int E, int top, int has_gate, cudaStream_t stream) {
  return gb_moe_topk_mode(z, ldz, bias, idx, wts, sg, ntok, E, top, has_gate, 0, stream);
}

// w_gu: [E, 2 ff, width] (an expert's gate rows, then its up rows); ws_gu: [2 ffs, width] or null;
// y: [ntok, slots, ffmax], slots = top (+ 1 with a shared expert), ffmax = max(ff, ffs).
GB_EXPORT int gb_moe_gate_up(const void* h, long long ldh, int dtype, const int* idx, const void* w_gu, const void* ws_gu,
                             void* y, int ntok, int width, int ff, int ffs, int top, float limit, float limit_s,
                             float alpha, float shift, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int slots = top + (ws_gu ? 1 : 0), ffmax = ff > ffs ? ff : ffs;
  if (width <= 0 || ffmax <= 0 || slots <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok * slots, (ffmax + FEATS - 1) / FEATS);
  if (dtype == GB_F32)
    gb_launch(moe_gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, ldh, idx, (const float*)w_gu,
              (const float*)ws_gu, (float*)y, width, ff, ffs, ffmax, top, slots, limit, limit_s, alpha, shift);
  else if (dtype == GB_BF16)
    gb_launch(moe_gate_up_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)h, ldh, idx, (const bf16*)w_gu,
              (const bf16*)ws_gu, (bf16*)y, width, ff, ffs, ffmax, top, slots, limit, limit_s, alpha, shift);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// Experts without a gate: w_up [E, ff, width]; y: [ntok, top, ff] = gelu(up h) of every chosen expert.
GB_EXPORT int gb_moe_up(const void* h, long long ldh, int dtype, const int* idx, const void* w_up, void* y, int ntok, int width,
                        int ff, int top, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (width <= 0 || ff <= 0 || top <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok * top, (ff + FEATS - 1) / FEATS);
  if (dtype == GB_F32)
    gb_launch(moe_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)h, ldh, idx, (const float*)w_up, (float*)y,
              width, ff, top);
  else if (dtype == GB_BF16)
    gb_launch(moe_up_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)h, ldh, idx, (const bf16*)w_up, (bf16*)y, width,
              ff, top);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// w_d: [E, width, ff]; ws_d: [width, ffs] or null; rows: float32 scratch [ntok, slots, width];
// residual: float32 [ntok, width] rows ldr apart.
GB_EXPORT int gb_moe_down(const void* y, int dtype, const int* idx, const float* wts, const float* sg, const void* w_d,
                          const void* ws_d, float* rows, float* residual, long long ldr, int ntok, int width, int ff, int ffs,
                          int top, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int slots = top + (ws_d ? 1 : 0), ffmax = ff > ffs ? ff : ffs;
  if (width <= 0 || ffmax <= 0 || slots <= 0) return GB_ERR_SIZE;
  const size_t smem = (size_t)ffmax * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_SIZE;
  dim3 grid(ntok * slots, (width + FEATS - 1) / FEATS);
  if (dtype == GB_F32)
    gb_launch(moe_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)y, idx, wts, sg, (const float*)w_d,
              (const float*)ws_d, rows, width, ff, ffs, ffmax, top, slots);
  else if (dtype == GB_BF16)
    gb_launch(moe_down_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)y, idx, wts, sg, (const bf16*)w_d,
              (const bf16*)ws_d, rows, width, ff, ffs, ffmax, top, slots);
  else
    return GB_ERR_DTYPE;
  gb_launch(moe_sum_kernel, dim3(ntok, (width + 1023) / 1024), dim3(256), 0, stream, (const float*)rows, residual, ldr, width,
            slots);
  return gb_launch_status();
}
