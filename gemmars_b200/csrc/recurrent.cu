// Kernels of the mixers that carry a fixed-size state from token to token: the short causal
// filter over time, the gated delta rule, the selective state-space recurrence with a scalar
// decay per head, and the gated RMS norm over groups of channels that follows them.
//
// A step's tokens are packed; sequence b owns rows cu[b] .. cu[b+1]-1 and the state row
// seq_slot[b].  Every kernel walks a sequence's rows in order on the device, so a whole prompt, a
// part of one and a single token run the same arithmetic, and a captured step needs no host.
// Rows that pad a captured step carry the spare slot, whose state row nobody reads.
//
// States and everything that enters a recurrence are float32: decays, step sizes, gates of the
// recurrence, unit norms.  Inputs are the float32 results of the projections.
#include "common.cuh"

constexpr int MAX_TAPS = 8;
enum { ACT_NONE = 0, ACT_SILU = 1 };

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ short causal filter
// y[t, c] = act(bias[c] + sum_j taps[c, j] * u[t - (K-1) + j, c]); rows before the step's first
// row of the sequence come from the K-1 rows kept in the state (oldest first), which are zero
// for a new sequence.
template <typename T>
__device__ __forceinline__ float filter_input(const T* __restrict__ u, long long ldu, int row0, int local,
                                              const float* __restrict__ hist, int C, int c, int K) {
  return local >= 0 ? to_f32(u[(size_t)(row0 + local) * ldu + c]) : hist[(size_t)(K - 1 + local) * C + c];
}

// A thread works one channel over `per` consecutive rows of the packed step and keeps the filter's
// window in registers, so a row costs one load, K multiply-adds and one store (with a thread a row
// and the window read again for every tap, the kernel was bound by the instructions of its index
// arithmetic: 231 a row, 0.17 of the memory's rate).  Where the rows pass from one sequence to the
// next, the window is read anew from the next sequence's memory.  A row's sums are taken in the
// same order whatever `per` is.
template <typename T, typename O>
__global__ void __launch_bounds__(256) short_filter_kernel(const T* __restrict__ u, long long ldu, const float* __restrict__ taps,
                                                          const float* __restrict__ bias, const float* __restrict__ state,
                                                          const int* __restrict__ cu, const int* __restrict__ tok_seq,
                                                          const int* __restrict__ seq_slot, O* __restrict__ out, long long ldo,
                                                          int ntok, int per, int C, int K, int act) {
  pdl_release_next();
  pdl_wait_prior();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float w[MAX_TAPS], win[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) w[j] = j < K ? taps[(size_t)c * K + j] : 0.f;
  const float b0 = bias ? bias[c] : 0.f;
  const int first = blockIdx.x * per, end = min(first + per, ntok);
  int b = tok_seq[first], row0 = cu[b], next_start = cu[b + 1];
  {
    const float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      win[j] = j < K - 1 ? filter_input(u, ldu, row0, first - row0 - (K - 1) + j, hist, C, c, K) : 0.f;
  }
  const T* in = u + (size_t)first * ldu + c;
  O* o = out + (size_t)first * ldo + c;
  for (int t = first; t < end; ++t, in += ldu, o += ldo) {
    if (t == next_start) {                      // the next sequence of the step starts here
      ++b;
      next_start = cu[b + 1];
      const float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
#pragma unroll
      for (int j = 0; j < MAX_TAPS - 1; ++j) win[j] = j < K - 1 ? hist[(size_t)j * C + c] : 0.f;
    }
    const float now = to_f32(*in);
    float acc = b0;
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < K - 1) acc = fmaf(w[j], win[j], acc);
    acc = fmaf(taps[(size_t)c * K + K - 1], now, acc);
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < K - 1) win[j] = j + 1 < K - 1 ? win[j + 1] : now;
    if (act == ACT_SILU) acc = silu_f(acc);
    *o = from_f32<O>(acc);
  }
}

// The state after the step: the last K-1 inputs of the sequence, old rows shifted where the step
// brought fewer than K-1.
template <typename T>
__global__ void __launch_bounds__(256) short_filter_state_kernel(const T* __restrict__ u, long long ldu, float* __restrict__ state,
                                                                const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                                                int C, int K) {
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row0 = cu[b], n = cu[b + 1] - row0;
  float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
  float next[MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < K - 1) next[i] = filter_input(u, ldu, row0, n - (K - 1) + i, hist, C, c, K);
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < K - 1) hist[(size_t)i * C + c] = next[i];
}

// A step of single tokens: the filter and its memory in one kernel, a thread per (sequence,
// channel), which alone reads and writes that channel's memory.  The sums are taken in the order
// of the kernel above, so a token gets the same bits whichever kernel ran it.
template <typename T, typename O>
__global__ void __launch_bounds__(256) short_filter_single_kernel(const T* __restrict__ u, long long ldu, const float* __restrict__ taps,
                                                                 const float* __restrict__ bias, float* __restrict__ state,
                                                                 const int* __restrict__ seq_slot, O* __restrict__ out,
                                                                 long long ldo, int C, int K, int act) {
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float* hist = state + (size_t)seq_slot[b] * (K - 1) * C;
  const float now = to_f32(u[(size_t)b * ldu + c]);
  float acc = bias ? bias[c] : 0.f;
  float held[MAX_TAPS - 1];
#pragma unroll
  for (int j = 0; j < MAX_TAPS - 1; ++j)
    if (j < K - 1) {
      held[j] = hist[(size_t)j * C + c];
      acc = fmaf(taps[(size_t)c * K + j], held[j], acc);
    }
  acc = fmaf(taps[(size_t)c * K + K - 1], now, acc);
  if (act == ACT_SILU) acc = silu_f(acc);
  out[(size_t)b * ldo + c] = from_f32<O>(acc);
#pragma unroll
  for (int j = 0; j < MAX_TAPS - 1; ++j)
    if (j < K - 1) hist[(size_t)j * C + c] = j + 1 < K - 1 ? held[j + 1] : now;
}

GB_EXPORT int gb_short_filter(const void* u, int in_dtype, long long ldu, const float* taps, const float* bias, float* state,
                              const int* cu, const int* tok_seq, const int* seq_slot, void* out, int out_dtype, long long ldo,
                              int ntok, int nseq, int C, int K, int act, int update_state, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (K < 1 || K > MAX_TAPS || C <= 0) return GB_ERR_SIZE;
  const int per = ntok >= 512 ? 16 : 1;        // rows a thread walks: a prompt's, or one of a small step
  dim3 grid((ntok + per - 1) / per, (C + 255) / 256), sgrid(nseq, (C + 255) / 256);
  if (ntok == nseq && update_state && K > 1) {     // every sequence brings one token
#define GB_SINGLE(T, O)                                                                                                     \
  gb_launch(short_filter_single_kernel<T, O>, sgrid, 256, 0, stream, (const T*)u, ldu, taps, bias, state, seq_slot, (O*)out, ldo, \
            C, K, act)
    if (in_dtype == GB_F32 && out_dtype == GB_F32) GB_SINGLE(float, float);
    else if (in_dtype == GB_F32 && out_dtype == GB_BF16) GB_SINGLE(float, bf16);
    else if (in_dtype == GB_BF16 && out_dtype == GB_BF16) GB_SINGLE(bf16, bf16);
    else if (in_dtype == GB_BF16 && out_dtype == GB_F32) GB_SINGLE(bf16, float);
    else return GB_ERR_DTYPE;
#undef GB_SINGLE
    return gb_launch_status();
  }
#define GB_FILTER(T, O)                                                                                                   \
  gb_launch(short_filter_kernel<T, O>, grid, 256, 0, stream, (const T*)u, ldu, taps, bias, (const float*)state, cu, tok_seq, \
            seq_slot, (O*)out, ldo, ntok, per, C, K, act)
  if (in_dtype == GB_F32 && out_dtype == GB_F32) GB_FILTER(float, float);
  else if (in_dtype == GB_F32 && out_dtype == GB_BF16) GB_FILTER(float, bf16);
  else if (in_dtype == GB_BF16 && out_dtype == GB_BF16) GB_FILTER(bf16, bf16);
  else if (in_dtype == GB_BF16 && out_dtype == GB_F32) GB_FILTER(bf16, float);
  else return GB_ERR_DTYPE;
#undef GB_FILTER
  if (update_state && K > 1) {
    if (in_dtype == GB_F32)
      gb_launch(short_filter_state_kernel<float>, sgrid, 256, 0, stream, (const float*)u, ldu, state, cu, seq_slot, C, K);
    else
      gb_launch(short_filter_state_kernel<bf16>, sgrid, 256, 0, stream, (const bf16*)u, ldu, state, cu, seq_slot, C, K);
  }
  return gb_launch_status();
}

// Only the state update (for a caller whose own kernel has applied the filter).
GB_EXPORT int gb_short_filter_state(const void* u, int in_dtype, long long ldu, float* state, const int* cu,
                                    const int* seq_slot, int nseq, int C, int K, cudaStream_t stream) {
  if (nseq <= 0 || K <= 1) return 0;
  if (K > MAX_TAPS || C <= 0) return GB_ERR_SIZE;
  dim3 sgrid(nseq, (C + 255) / 256);
  if (in_dtype == GB_F32)
    gb_launch(short_filter_state_kernel<float>, sgrid, 256, 0, stream, (const float*)u, ldu, state, cu, seq_slot, C, K);
  else if (in_dtype == GB_BF16)
    gb_launch(short_filter_state_kernel<bf16>, sgrid, 256, 0, stream, (const bf16*)u, ldu, state, cu, seq_slot, C, K);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// ------------------------------------------------------------------ gated delta rule
// The state of a head is a matrix S [dim, vdim].  A block is 32 columns of one (sequence, head);
// a column is worked by P lanes side by side, each holding 32 of the column's dims in registers
// (dim <= 32 P, zeros beyond).  In memory a head's state is kept in the order the lanes read it,
// 16 bytes a lane and a warp's lanes side by side: element (d, col), d = 32 part + 4 r + e, lies at
// ((r * vdim + col) * P + part) * 4 + e  (8 * vdim * P * 4 floats a head).
// Per token, with k^ = k / sqrt(|k|^2 + 1e-6), q^ = q / sqrt(|q|^2 + 1e-6) * qscale,
// beta = sigmoid(bl), g = exp(-exp(A_log) * softplus(al + dt_bias)):
//   S <- g S;  u = beta (v - S^T k^);  S <- S + k^ u^T;  y = S^T q^
// The two products with the old state are taken in one pass (y = g S_old^T q^ + (k^ . q^) u) and
// meet over the P lanes by shuffles.  Tokens come into shared memory eight at a time by
// asynchronous copies, a group ahead of the one being worked; what does not depend on the state
// (the norms of k and q, k . q, beta, the decay) is worked out for the whole group at once, a
// token a warp, so that the walk from token to token is the state's arithmetic alone.
constexpr int SLICE = 32;   // dims of a column that one lane holds
constexpr int GROUP = 8;    // tokens brought in together
// A lane's 32 dims of k, q, B or C start 36 floats after its neighbour's: the P lanes of a column
// read their 16 bytes from different banks (128 bytes apart they would all hit the same four).
__device__ __forceinline__ int padded(int i) { return i + (i >> 5) * 4; }
constexpr int padded_size(int lanes) { return lanes * (SLICE + 4); }

template <int P>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = P / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// CH: the decay is a vector per head, one number per key channel, given as it is (``a_logit`` then
// holds the decays, rows of ``lda`` floats, head h at h * D): row d of S is multiplied by g_d before
// the token's read and write.  A_log and dt_bias are not read.
template <int P, bool CH>
__global__ void __launch_bounds__(32 * P) delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                           const float* __restrict__ v, long long ld,
                                                           const float* __restrict__ beta_logit, const float* __restrict__ a_logit,
                                                           long long ldg, long long lda, const float* __restrict__ A_log,
                                                           const float* __restrict__ dt_bias, float* __restrict__ state,
                                                           const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                                           float* __restrict__ y, int H, int G, int D, int V, float qscale) {
  constexpr int DP = P * SLICE;
  constexpr int GRP = (CH && P == 8) ? GROUP / 2 : GROUP;   // tokens a group: what 48 KB of shared memory hold
  __shared__ __align__(16) float kq[2][GRP][CH ? 3 : 2][padded_size(P)];   // [buffer][token][k | q (| decay)][dims, padded]
  __shared__ float vs[2][GRP][32], gates[2][GRP][2];
  __shared__ float pre[GRP][4];                       // per token: decay, 1/|k|, beta, (k^ . q^); then decay * qscale/|q|
  __shared__ float pre_q[GRP];
  pdl_wait_prior();
  const int b = blockIdx.x, head = blockIdx.y, g = head / (H / G), tid = threadIdx.x;
  const int col = blockIdx.z * 32 + tid / P, part = tid % P, lane = tid & 31, warp = tid >> 5;
  const bool live = col < V;
  const int t0 = cu[b], t1 = cu[b + 1];
  float4* Sg = (float4*)(state + ((size_t)seq_slot[b] * H + head) * 8 * V * P * 4);
  float S[SLICE];
#pragma unroll
  for (int r = 0; r < SLICE / 4; ++r) {
    const float4 s4 = live ? Sg[((size_t)r * V + col) * P + part] : make_float4(0.f, 0.f, 0.f, 0.f);
    S[4 * r] = s4.x; S[4 * r + 1] = s4.y; S[4 * r + 2] = s4.z; S[4 * r + 3] = s4.w;
  }
  const float rate = CH ? 0.f : expf(A_log[head]), dtb = CH ? 0.f : dt_bias[head];
  if (tid >= D)      // the dims beyond the head's are zeros, written once
    for (int j = 0; j < 2 * GRP; ++j)
      for (int a = 0; a < (CH ? 3 : 2); ++a) kq[j / GRP][j % GRP][a][padded(tid)] = 0.f;
  // every thread brings one dim of k and of q of every token of a group
  auto bring = [&](int first, int buf) {
    for (int j = 0; j < GRP && first + j < t1; ++j) {
      const size_t t = first + j;
      if (tid < D) {
        copy_async4(&kq[buf][j][0][padded(tid)], k + t * ld + g * D + tid);
        copy_async4(&kq[buf][j][1][padded(tid)], q + t * ld + g * D + tid);
        if (CH) copy_async4(&kq[buf][j][2][padded(tid)], a_logit + t * lda + head * D + tid);
      }
      if (live && part == 0) copy_async4(&vs[buf][j][tid / P], v + t * ld + head * V + col);
      if (tid == 0) copy_async4(&gates[buf][j][0], beta_logit + t * ldg + head);
      if (!CH && tid == 1) copy_async4(&gates[buf][j][1], a_logit + t * lda + head);
    }
    copy_async_commit();
  };
  bring(t0, 0);
  for (int first = t0; first < t1; first += GRP) {
    const int buf = ((first - t0) / GRP) & 1;
    if (first + GRP < t1) {
      bring(first + GRP, buf ^ 1);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const int n = min(GRP, t1 - first);
    for (int j = warp; j < n; j += P) {       // a token a warp: what the state has no part in
      float kk = 0.f, qq = 0.f, kdq = 0.f;
      for (int i = lane; i < DP; i += 32) {
        const float kv = kq[buf][j][0][padded(i)], qv = kq[buf][j][1][padded(i)];
        kk = fmaf(kv, kv, kk); qq = fmaf(qv, qv, qq); kdq = fmaf(kv, qv, kdq);
      }
      kk = warp_sum(kk); qq = warp_sum(qq); kdq = warp_sum(kdq);
      if (lane == 0) {
        const float inv_k = 1.0f / sqrtf(kk + 1e-6f), inv_q = qscale / sqrtf(qq + 1e-6f);
        const float decay = CH ? 1.0f : expf(-rate * softplus_f(gates[buf][j][1] + dtb));
        pre[j][0] = decay; pre[j][1] = inv_k; pre[j][2] = sigmoid_f(gates[buf][j][0]); pre[j][3] = kdq * inv_k * inv_q;
        pre_q[j] = decay * inv_q;
      }
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float4* ks = (const float4*)(kq[buf][j][0] + part * (SLICE + 4));
      const float4* qs = (const float4*)(kq[buf][j][1] + part * (SLICE + 4));
      float4 kheld[SLICE / 4];              // k is used twice: kept between the read and the write of S
      float sk = 0.f, sk2 = 0.f, sq = 0.f, sq2 = 0.f;
#pragma unroll
      for (int r = 0; r < SLICE / 4; ++r) {
        const float4 kv = kheld[r] = ks[r], qv = qs[r];
        if (CH) {                             // the rows' own decays first: what follows reads the decayed state
          const float4 gv = ((const float4*)(kq[buf][j][CH ? 2 : 0] + part * (SLICE + 4)))[r];
          S[4 * r] *= gv.x; S[4 * r + 1] *= gv.y; S[4 * r + 2] *= gv.z; S[4 * r + 3] *= gv.w;
        }
        sk = fmaf(S[4 * r], kv.x, sk); sk2 = fmaf(S[4 * r + 1], kv.y, sk2); sk = fmaf(S[4 * r + 2], kv.z, sk); sk2 = fmaf(S[4 * r + 3], kv.w, sk2);
        sq = fmaf(S[4 * r], qv.x, sq); sq2 = fmaf(S[4 * r + 1], qv.y, sq2); sq = fmaf(S[4 * r + 2], qv.z, sq); sq2 = fmaf(S[4 * r + 3], qv.w, sq2);
      }
      sk = lanes_sum<P>(sk + sk2);
      sq = lanes_sum<P>(sq + sq2);
      const float decay = pre[j][0], inv_k = pre[j][1];
      const float u = pre[j][2] * ((live ? vs[buf][j][tid / P] : 0.f) - decay * inv_k * sk);
      const float ku = inv_k * u;
#pragma unroll
      for (int r = 0; r < SLICE / 4; ++r) {
        const float4 kv = kheld[r];
        S[4 * r] = fmaf(kv.x, ku, decay * S[4 * r]);
        S[4 * r + 1] = fmaf(kv.y, ku, decay * S[4 * r + 1]);
        S[4 * r + 2] = fmaf(kv.z, ku, decay * S[4 * r + 2]);
        S[4 * r + 3] = fmaf(kv.w, ku, decay * S[4 * r + 3]);
      }
      if (live && part == 0) y[(size_t)(first + j) * H * V + head * V + col] = fmaf(pre[j][3], u, pre_q[j] * sq);
    }
    __syncthreads();   // the group after next is brought into this buffer; pre is written again
  }
  // only now may the kernel after this one start: its waiting blocks would take the room of this
  // kernel's few warps, which are a chain from token to token
  pdl_release_next();
  if (live) {
#pragma unroll
    for (int r = 0; r < SLICE / 4; ++r)
      Sg[((size_t)r * V + col) * P + part] = make_float4(S[4 * r], S[4 * r + 1], S[4 * r + 2], S[4 * r + 3]);
  }
}

// A scan of few blocks (a prompt of one or two sequences) is launched without the attribute that lets
// it start under the kernel before it.  Started early, its blocks are placed on whichever SMs have room
// at that moment, several to an SM, and then share that SM's shared-memory bandwidth for the whole walk:
// measured, a 2,048-token prompt of four layers took 8.5 ms against 6.4 when the kernel before the scans
// became one of fewer, longer blocks.  Started when the GPU is idle, the blocks spread one to an SM.
template <typename Kernel, typename... Args>
static inline void launch_scan(Kernel kernel, dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
  if ((size_t)grid.x * grid.y * grid.z > 2 * 148) {
    gb_launch(kernel, grid, block, 0, stream, static_cast<Args&&>(args)...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}

static inline int lanes_for(int dims) { return dims <= SLICE ? 1 : (dims <= 2 * SLICE ? 2 : (dims <= 4 * SLICE ? 4 : 8)); }

// Floats of one head's state for columns of ``dims`` (what a caller allocates per slot and head).
GB_EXPORT int gb_state_floats(int dims, int V) { return 8 * V * lanes_for(dims) * 4; }

// state: [slots, H, gb_state_floats(D, V)] float32, in the order described above.
GB_EXPORT int gb_delta_rule(const float* q, const float* k, const float* v, long long ld, const float* beta_logit,
                            const float* a_logit, long long ldg, const float* A_log, const float* dt_bias, float* state,
                            const int* cu, const int* seq_slot, float* y, int nseq, int H, int G, int D, int V, float qscale,
                            cudaStream_t stream) {
  if (nseq <= 0) return 0;
  if (G <= 0 || H % G || V <= 0 || D <= 0 || D > 8 * SLICE || ((uintptr_t)state & 15)) return GB_ERR_SIZE;
  dim3 grid(nseq, H, (V + 31) / 32);
#define GB_DELTA(P)                                                                                                    \
  launch_scan(delta_rule_kernel<P, false>, grid, 32 * P, stream, q, k, v, ld, beta_logit, a_logit, ldg, ldg, A_log, dt_bias, state, cu, \
              seq_slot, y, H, G, D, V, qscale)
  switch (lanes_for(D)) {
    case 1: GB_DELTA(1); break;
    case 2: GB_DELTA(2); break;
    case 4: GB_DELTA(4); break;
    default: GB_DELTA(8);
  }
#undef GB_DELTA
  return gb_launch_status();
}

// The delta rule with a decay per head and key channel: decay [ntok, H * D] rows of ldd floats, the
// numbers g in (0, 1] themselves; beta_logit rows of ldb floats.  The rest as gb_delta_rule.
GB_EXPORT int gb_channel_delta_rule(const float* q, const float* k, const float* v, long long ld, const float* beta_logit,
                                    long long ldb, const float* decay, long long ldd, float* state, const int* cu,
                                    const int* seq_slot, float* y, int nseq, int H, int G, int D, int V, float qscale,
                                    cudaStream_t stream) {
  if (nseq <= 0) return 0;
  if (G <= 0 || H % G || V <= 0 || D <= 0 || D > 8 * SLICE || ((uintptr_t)state & 15) || !decay) return GB_ERR_SIZE;
  dim3 grid(nseq, H, (V + 31) / 32);
#define GB_DELTA(P)                                                                                                    \
  launch_scan(delta_rule_kernel<P, true>, grid, 32 * P, stream, q, k, v, ld, beta_logit, decay, ldb, ldd, (const float*)nullptr, \
              (const float*)nullptr, state, cu, seq_slot, y, H, G, D, V, qscale)
  switch (lanes_for(D)) {
    case 1: GB_DELTA(1); break;
    case 2: GB_DELTA(2); break;
    case 4: GB_DELTA(4); break;
    default: GB_DELTA(8);
  }
#undef GB_DELTA
  return gb_launch_status();
}

// ------------------------------------------------------------------ selective state space, scalar decay per head
// The state of a head is S [n_state, vdim]; blocks, columns, lanes and the order in memory as
// above (n_state <= 32 P).  Per token, with dt = softplus(dt_raw + dt_bias):
//   S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x.
template <int P>
__global__ void __launch_bounds__(32 * P) ssd_scan_kernel(const float* __restrict__ x, const float* __restrict__ Bm,
                                                         const float* __restrict__ Cm, long long ld,
                                                         const float* __restrict__ dt_raw, long long ldd,
                                                         const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                         const float* __restrict__ skip, float* __restrict__ state,
                                                         const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                                         float* __restrict__ y, int H, int G, int N, int V) {
  __shared__ __align__(16) float bc[2][GROUP][2][padded_size(P)];   // [buffer][token][B | C][state dims, padded]
  __shared__ float xs[2][GROUP][32], steps[2][GROUP], pre[GROUP][2];
  pdl_wait_prior();
  const int b = blockIdx.x, head = blockIdx.y, g = head / (H / G), tid = threadIdx.x;
  const int col = blockIdx.z * 32 + tid / P, part = tid % P;
  const bool live = col < V;
  const int t0 = cu[b], t1 = cu[b + 1];
  float4* Sg = (float4*)(state + ((size_t)seq_slot[b] * H + head) * 8 * V * P * 4);
  float S[SLICE];
#pragma unroll
  for (int r = 0; r < SLICE / 4; ++r) {
    const float4 s4 = live ? Sg[((size_t)r * V + col) * P + part] : make_float4(0.f, 0.f, 0.f, 0.f);
    S[4 * r] = s4.x; S[4 * r + 1] = s4.y; S[4 * r + 2] = s4.z; S[4 * r + 3] = s4.w;
  }
  const float rate = expf(A_log[head]), dtb = dt_bias[head], dskip = skip[head];
  if (tid >= N)
    for (int j = 0; j < 2 * GROUP; ++j) bc[j / GROUP][j % GROUP][0][padded(tid)] = bc[j / GROUP][j % GROUP][1][padded(tid)] = 0.f;
  auto bring = [&](int first, int buf) {
    for (int j = 0; j < GROUP && first + j < t1; ++j) {
      const size_t t = first + j;
      if (tid < N) {
        copy_async4(&bc[buf][j][0][padded(tid)], Bm + t * ld + g * N + tid);
        copy_async4(&bc[buf][j][1][padded(tid)], Cm + t * ld + g * N + tid);
      }
      if (live && part == 0) copy_async4(&xs[buf][j][tid / P], x + t * ld + head * V + col);
      if (tid == 0) copy_async4(&steps[buf][j], dt_raw + t * ldd + head);
    }
    copy_async_commit();
  };
  bring(t0, 0);
  for (int first = t0; first < t1; first += GROUP) {
    const int buf = ((first - t0) / GROUP) & 1;
    if (first + GROUP < t1) {
      bring(first + GROUP, buf ^ 1);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const int n = min(GROUP, t1 - first);
    if (tid < n) {                            // step sizes and decays of the group, a token a thread
      const float dt = softplus_f(steps[buf][tid] + dtb);
      pre[tid][0] = dt;
      pre[tid][1] = expf(-rate * dt);
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float4* Bs = (const float4*)(bc[buf][j][0] + part * (SLICE + 4));
      const float4* Cs = (const float4*)(bc[buf][j][1] + part * (SLICE + 4));
      const float xv = live ? xs[buf][j][tid / P] : 0.f;
      const float decay = pre[j][1], dx = pre[j][0] * xv;
      float acc = 0.f, acc2 = 0.f;
#pragma unroll
      for (int r = 0; r < SLICE / 4; ++r) {
        const float4 bv = Bs[r], cv = Cs[r];
        S[4 * r] = fmaf(bv.x, dx, decay * S[4 * r]);         acc = fmaf(S[4 * r], cv.x, acc);
        S[4 * r + 1] = fmaf(bv.y, dx, decay * S[4 * r + 1]); acc2 = fmaf(S[4 * r + 1], cv.y, acc2);
        S[4 * r + 2] = fmaf(bv.z, dx, decay * S[4 * r + 2]); acc = fmaf(S[4 * r + 2], cv.z, acc);
        S[4 * r + 3] = fmaf(bv.w, dx, decay * S[4 * r + 3]); acc2 = fmaf(S[4 * r + 3], cv.w, acc2);
      }
      acc = lanes_sum<P>(acc + acc2);
      if (live && part == 0) y[(size_t)(first + j) * H * V + head * V + col] = fmaf(dskip, xv, acc);
    }
    __syncthreads();
  }
  // only now may the kernel after this one start: its waiting blocks would take the room of this
  // kernel's few warps, which are a chain from token to token
  pdl_release_next();
  if (live) {
#pragma unroll
    for (int r = 0; r < SLICE / 4; ++r)
      Sg[((size_t)r * V + col) * P + part] = make_float4(S[4 * r], S[4 * r + 1], S[4 * r + 2], S[4 * r + 3]);
  }
}

// state: [slots, H, gb_state_floats(N, V)] float32.
GB_EXPORT int gb_ssd_scan(const float* x, const float* Bm, const float* Cm, long long ld, const float* dt_raw, long long ldd,
                          const float* A_log, const float* dt_bias, const float* skip, float* state, const int* cu,
                          const int* seq_slot, float* y, int nseq, int H, int G, int N, int V, cudaStream_t stream) {
  if (nseq <= 0) return 0;
  if (G <= 0 || H % G || V <= 0 || N <= 0 || N > 8 * SLICE || ((uintptr_t)state & 15)) return GB_ERR_SIZE;
  dim3 grid(nseq, H, (V + 31) / 32);
#define GB_SSD(P)                                                                                                       \
  launch_scan(ssd_scan_kernel<P>, grid, 32 * P, stream, x, Bm, Cm, ld, dt_raw, ldd, A_log, dt_bias, skip, state, cu, seq_slot, y, \
              H, G, N, V)
  switch (lanes_for(N)) {
    case 1: GB_SSD(1); break;
    case 2: GB_SSD(2); break;
    case 4: GB_SSD(4); break;
    default: GB_SSD(8);
  }
#undef GB_SSD
  return gb_launch_status();
}

// ------------------------------------------------------------------ gated RMS norm over groups of channels
// Row t of y [T, n] is cut into groups of gs channels, each divided by its own root mean square;
// channel i is weighed by w[i % wn] and gated by silu(gate[t, i]) (gate_act 0) or sigmoid(gate[t, i])
// (gate_act 1).  gate_first: the gate is multiplied in before the statistics are taken (the norm
// sees the gated values), else after.
__device__ __forceinline__ float gate_f(float z, int act) { return act ? sigmoid_f(z) : silu_f(z); }
template <typename O>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                              long long ldgate, const float* __restrict__ w, int wn,
                                                              O* __restrict__ out, int n, int gs, float eps, int gate_first,
                                                              float out_scale, int gate_act) {
  __shared__ float scratch[33];
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, base = blockIdx.y * gs;
  const float* row = y + (size_t)t * n + base;
  const float* grow = gate + (size_t)t * ldgate + base;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float val = gate_first ? row[i] * gate_f(grow[i], gate_act) : row[i];
    ss = fmaf(val, val, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float gt = gate_f(grow[i], gate_act);
    const float val = gate_first ? row[i] * gt * inv * w[(base + i) % wn] : row[i] * inv * w[(base + i) % wn] * gt;
    out[(size_t)t * n + base + i] = from_f32<O>(val * out_scale);
  }
}

// The same for groups of at most 32 E channels (E = 2 or 4): a warp a group (eight groups a block),
// the sum by shuffles, so that a token's row is not cut into blocks of one or two warps.
template <typename O, int E>
__global__ void __launch_bounds__(256) gated_group_norm_warp_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                                   long long ldgate, const float* __restrict__ w, int wn,
                                                                   O* __restrict__ out, int n, int gs, float eps, int gate_first,
                                                                   float out_scale, int gate_act) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, group = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (group * gs >= n) return;
  const int base = group * gs;
  const float* row = y + (size_t)t * n + base;
  const float* grow = gate + (size_t)t * ldgate + base;
  float val[E], gt[E], ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = lane + 32 * e;
    val[e] = i < gs ? row[i] : 0.f;
    gt[e] = i < gs ? gate_f(grow[i], gate_act) : 0.f;
    if (gate_first) val[e] *= gt[e];
    ss = fmaf(val[e], val[e], ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = lane + 32 * e;
    if (i >= gs) continue;
    const float res = gate_first ? val[e] * inv * w[(base + i) % wn] : val[e] * inv * w[(base + i) % wn] * gt[e];
    out[(size_t)t * n + base + i] = from_f32<O>(res * out_scale);
  }
}

GB_EXPORT int gb_gated_group_norm_act(const float* y, const float* gate, long long ldgate, const float* w, int wn, void* out,
                                      int out_dtype, int ntok, int n, int gs, float eps, int gate_first, float out_scale,
                                      int gate_act, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (gs <= 0 || n % gs || wn <= 0) return GB_ERR_SIZE;
  if (out_dtype != GB_F32 && out_dtype != GB_BF16) return GB_ERR_DTYPE;
  if (gs <= 128) {
    dim3 wgrid(ntok, (n / gs + 7) / 8);
#define GB_NORM_WARP(O, E)                                                                                              \
  gb_launch(gated_group_norm_warp_kernel<O, E>, wgrid, 256, 0, stream, y, gate, ldgate, w, wn, (O*)out, n, gs, eps, gate_first, \
            out_scale, gate_act)
    if (out_dtype == GB_F32) { if (gs <= 64) GB_NORM_WARP(float, 2); else GB_NORM_WARP(float, 4); }
    else { if (gs <= 64) GB_NORM_WARP(bf16, 2); else GB_NORM_WARP(bf16, 4); }
#undef GB_NORM_WARP
    return gb_launch_status();
  }
  dim3 grid(ntok, n / gs);
  const int threads = gs <= 32 ? 32 : (gs <= 64 ? 64 : 128);
  if (out_dtype == GB_F32)
    gb_launch(gated_group_norm_kernel<float>, grid, threads, 0, stream, y, gate, ldgate, w, wn, (float*)out, n, gs, eps,
              gate_first, out_scale, gate_act);
  else if (out_dtype == GB_BF16)
    gb_launch(gated_group_norm_kernel<bf16>, grid, threads, 0, stream, y, gate, ldgate, w, wn, (bf16*)out, n, gs, eps, gate_first,
              out_scale, gate_act);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

GB_EXPORT int gb_gated_group_norm(const float* y, const float* gate, long long ldgate, const float* w, int wn, void* out,
                                  int out_dtype, int ntok, int n, int gs, float eps, int gate_first, float out_scale,
                                  cudaStream_t stream) {
  return gb_gated_group_norm_act(y, gate, ldgate, w, wn, out, out_dtype, ntok, n, gs, eps, gate_first, out_scale, 0, stream);
}

// ------------------------------------------------------------------ mixes with the token before
// out[s, t, c] = x[t, c] + (x[t - 1, c] - x[t, c]) * mu[s, c] for each of the n_mix rows of mu: every
// consumer reads its own blend of a token's row and the row before it in the same sequence.  The
// row before a step's first row of a sequence is the state's (float32 [slots, C], zeros for a new
// sequence); afterwards the state holds the step's last row of the sequence.  In a step of single
// tokens (`single`) the thread that read the state writes it; otherwise shift_state_kernel follows.
template <typename T>
__global__ void __launch_bounds__(256) shift_mix_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ mu,
                                                       float* __restrict__ state, const int* __restrict__ cu,
                                                       const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                                       T* __restrict__ out, int ntok, int C, int n_mix, int single) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, b = tok_seq[t];
  const bool first = t == cu[b];
  float* st = state + (size_t)seq_slot[b] * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const float cur = to_f32(x[(size_t)t * ldx + c]);
    const float before = first ? st[c] : to_f32(x[(size_t)(t - 1) * ldx + c]);
    const float d = before - cur;
    for (int s = 0; s < n_mix; ++s) out[((size_t)s * ntok + t) * C + c] = from_f32<T>(fmaf(d, mu[(size_t)s * C + c], cur));
    if (single) st[c] = cur;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) shift_state_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ state,
                                                         const int* __restrict__ cu, const int* __restrict__ seq_slot, int C) {
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x, last = cu[b + 1] - 1;
  if (last < cu[b]) return;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x)
    state[(size_t)seq_slot[b] * C + c] = to_f32(x[(size_t)last * ldx + c]);
}

// mu: [n_mix, C] float32; out: [n_mix, ntok, C] in x's type; state: [slots, C] float32.
GB_EXPORT int gb_shift_mix(const void* x, int dtype, long long ldx, const float* mu, float* state, const int* cu,
                           const int* tok_seq, const int* seq_slot, void* out, int ntok, int nseq, int C, int n_mix,
                           cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (C <= 0 || n_mix <= 0 || nseq <= 0) return GB_ERR_SIZE;
  const int single = ntok == nseq;
  const dim3 grid(ntok, (C + 1023) / 1024), sgrid(nseq, (C + 1023) / 1024);
  if (dtype == GB_F32) {
    gb_launch(shift_mix_kernel<float>, grid, 256, 0, stream, (const float*)x, ldx, mu, state, cu, tok_seq, seq_slot, (float*)out,
              ntok, C, n_mix, single);
    if (!single) gb_launch(shift_state_kernel<float>, sgrid, 256, 0, stream, (const float*)x, ldx, state, cu, seq_slot, C);
  } else if (dtype == GB_BF16) {
    gb_launch(shift_mix_kernel<bf16>, grid, 256, 0, stream, (const bf16*)x, ldx, mu, state, cu, tok_seq, seq_slot, (bf16*)out,
              ntok, C, n_mix, single);
    if (!single) gb_launch(shift_state_kernel<bf16>, sgrid, 256, 0, stream, (const bf16*)x, ldx, state, cu, seq_slot, C);
  } else {
    return GB_ERR_DTYPE;
  }
  return gb_launch_status();
}

// ------------------------------------------------------------------ decay from a low-rank projection
// w[t, c] = exp(-exp(base[c] + sum_j W[c, j] tanh(z[t, j]))): the second half of a two-matrix decay
// whose first product z = W1 x is made by the framework's product in float32.  tanh, the sum, both
// exponentials and the result are float32.  A block is 128 channels by DEC_TOK tokens: a thread
// keeps a channel's sums for the block's tokens in registers and walks its row of W once, against
// tanh(z) of the tokens in shared memory (DEC_RC entries of the rank a pass).  Every sum runs over
// the rank in order with one accumulator, so the result does not depend on the tiling.
constexpr int DEC_TOK = 8, DEC_RC = 128;
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 a = *(const uint4*)p;
  const unsigned u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {      // a bfloat16 is the upper half of the float32 of the same value
    v[2 * e] = __uint_as_float(u[e] << 16);
    v[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
  }
}
// Other forms of the same two-step projection (``mode``), z going in as it is (no tanh):
//   LR_RATE:     exp(-exp(rate[c / rate_group]) * softplus(a + base[c]))   a step size per channel, a rate per group
//   LR_SIGMOID_ROOT: sigmoid(a + base[c])^(1 / tau) = exp(-softplus(-(a + base[c])) / tau)
//   LR_PLAIN:    a + base[c]
// with a = sum_j W[c, j] z[t, j]; base may be null (zeros).
enum { LR_TANH_EXPEXP = 0, LR_RATE = 1, LR_SIGMOID_ROOT = 2, LR_PLAIN = 3 };
template <typename T>
__global__ void __launch_bounds__(128) lowrank_decay_kernel(const float* __restrict__ z, long long ldz, int rank,
                                                           const T* __restrict__ W, const float* __restrict__ base,
                                                           float* __restrict__ w, int ntok, int C, int mode,
                                                           const float* __restrict__ rate, int rate_group, float inv_tau) {
  __shared__ __align__(16) float th[DEC_TOK][DEC_RC];      // tanh(z[t0 + tt, j0 + j]), zeros beyond the edges
  pdl_release_next();
  pdl_wait_prior();
  const int c = blockIdx.x * 128 + threadIdx.x, t0 = blockIdx.y * DEC_TOK;
  const int n = min(DEC_TOK, ntok - t0);
  const T* row = W + (size_t)min(c, C - 1) * rank;
  const bool vec = rank % 8 == 0 && ((uintptr_t)W & 15) == 0;
  float acc[DEC_TOK];
#pragma unroll
  for (int tt = 0; tt < DEC_TOK; ++tt) acc[tt] = 0.f;
  for (int j0 = 0; j0 < rank; j0 += DEC_RC) {
    const int nj = min(DEC_RC, rank - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < DEC_TOK * DEC_RC; i += 128) {
      const int tt = i / DEC_RC, j = i % DEC_RC;
      const float zin = (tt < n && j < nj) ? z[(size_t)(t0 + tt) * ldz + j0 + j] : 0.f;
      th[tt][j] = mode == LR_TANH_EXPEXP ? tanhf(zin) : zin;
    }
    __syncthreads();
    for (int j = 0; j < nj; j += 8) {
      float wv[8];
      if (vec) {         // rows start on 16-byte boundaries and hold a multiple of eight entries
        load8(row + j0 + j, wv);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = j + e < nj ? to_f32(row[j0 + j + e]) : 0.f;
      }
#pragma unroll
      for (int tt = 0; tt < DEC_TOK; ++tt) {
        const float4 h = *(const float4*)&th[tt][j], g = *(const float4*)&th[tt][j + 4];
        acc[tt] = fmaf(wv[0], h.x, acc[tt]);
        acc[tt] = fmaf(wv[1], h.y, acc[tt]);
        acc[tt] = fmaf(wv[2], h.z, acc[tt]);
        acc[tt] = fmaf(wv[3], h.w, acc[tt]);
        acc[tt] = fmaf(wv[4], g.x, acc[tt]);
        acc[tt] = fmaf(wv[5], g.y, acc[tt]);
        acc[tt] = fmaf(wv[6], g.z, acc[tt]);
        acc[tt] = fmaf(wv[7], g.w, acc[tt]);
      }
    }
  }
  if (c >= C) return;
  const float b = base ? base[c] : 0.f;
  const float rt = mode == LR_RATE ? expf(rate[c / rate_group]) : 0.f;
#pragma unroll
  for (int tt = 0; tt < DEC_TOK; ++tt)
    if (tt < n) {
      const float a = acc[tt] + b;
      float r;
      if (mode == LR_TANH_EXPEXP) r = expf(-expf(a));
      else if (mode == LR_RATE) r = expf(-rt * softplus_f(a));
      else if (mode == LR_SIGMOID_ROOT) r = expf(-softplus_f(-a) * inv_tau);
      else r = a;
      w[(size_t)(t0 + tt) * C + c] = r;
    }
}

// z: [ntok, rank] float32; W: [C, rank] float32 or bfloat16; base: [C]; w: [ntok, C] float32.
// The general form (see the modes above): z rows of ldz floats; rate [C / rate_group] for LR_RATE;
// tau for LR_SIGMOID_ROOT.
GB_EXPORT int gb_lowrank_map(const float* z, long long ldz, int rank, const void* W, int w_dtype, const float* base, float* w,
                             int ntok, int C, int mode, const float* rate, int rate_group, float tau, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (rank <= 0 || rank > 8192 || C <= 0 || mode < LR_TANH_EXPEXP || mode > LR_PLAIN) return GB_ERR_SIZE;
  if (mode == LR_RATE && (!rate || rate_group <= 0)) return GB_ERR_ARG;
  if (mode == LR_SIGMOID_ROOT && !(tau > 0.f)) return GB_ERR_ARG;
  if (mode == LR_TANH_EXPEXP && !base) return GB_ERR_ARG;
  const dim3 grid((C + 127) / 128, (ntok + DEC_TOK - 1) / DEC_TOK);
  if (grid.y > 65535) return GB_ERR_SIZE;
  const float inv_tau = mode == LR_SIGMOID_ROOT ? 1.0f / tau : 0.f;
  if (w_dtype == GB_F32)
    gb_launch(lowrank_decay_kernel<float>, grid, 128, 0, stream, z, ldz, rank, (const float*)W, base, w, ntok, C, mode, rate,
              rate_group, inv_tau);
  else if (w_dtype == GB_BF16)
    gb_launch(lowrank_decay_kernel<bf16>, grid, 128, 0, stream, z, ldz, rank, (const bf16*)W, base, w, ntok, C, mode, rate,
              rate_group, inv_tau);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

GB_EXPORT int gb_lowrank_decay(const float* z, int rank, const void* W, int w_dtype, const float* base, float* w, int ntok,
                               int C, cudaStream_t stream) {
  return gb_lowrank_map(z, rank, rank, W, w_dtype, base, w, ntok, C, LR_TANH_EXPEXP, nullptr, 1, 0.f, stream);
}

// ------------------------------------------------------------------ linear attention with a decay per key channel
// The state of a head is S [dim, vdim]; blocks, columns, lanes and the order in memory as for the
// delta rule (dim <= 32 P).  Per token, with w the decay of every key channel (0..1) and u a
// bonus per head and key channel that only the token itself gets:
//   y = (S + diag(u) k v^T)^T r = S^T r + (sum_d r_d u_d k_d) v;   S <- diag(w) S + k v^T
// The read-out sees the state as the tokens before left it.  Tokens come in groups of GR by
// asynchronous copies, a group ahead; the sum over r u k is taken for the group at once, a token
// a warp.  Everything is float32.
// AFTER (no bonus): the read-out follows the write, S <- diag(w) S + k v^T; y = S^T r, which is the
// recurrence of gated linear attention.
template <int P, int GR, bool AFTER>
__global__ void __launch_bounds__(32 * P) wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k,
                                                         const float* __restrict__ w, long long ld, long long ldw,
                                                         const float* __restrict__ v, long long ldv, const float* __restrict__ bonus, float* __restrict__ state,
                                                         const int* __restrict__ cu, const int* __restrict__ seq_slot,
                                                         float* __restrict__ y, int H, int D, int V, float yscale) {
  constexpr int DP = P * SLICE;
  __shared__ __align__(16) float rkw[2][GR][3][padded_size(P)];   // [buffer][token][r | k | w][dims, padded]
  __shared__ float vs[2][GR][32];
  __shared__ float us[padded_size(P)];
  __shared__ float ruk[GR];
  pdl_wait_prior();
  const int b = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int col = blockIdx.z * 32 + tid / P, part = tid % P, lane = tid & 31, warp = tid >> 5;
  const bool live = col < V;
  const int t0 = cu[b], t1 = cu[b + 1];
  float4* Sg = (float4*)(state + ((size_t)seq_slot[b] * H + head) * 8 * V * P * 4);
  float S[SLICE];
#pragma unroll
  for (int q = 0; q < SLICE / 4; ++q) {
    const float4 s4 = live ? Sg[((size_t)q * V + col) * P + part] : make_float4(0.f, 0.f, 0.f, 0.f);
    S[4 * q] = s4.x; S[4 * q + 1] = s4.y; S[4 * q + 2] = s4.z; S[4 * q + 3] = s4.w;
  }
  us[padded(tid)] = (!AFTER && tid < D) ? bonus[(size_t)head * D + tid] : 0.f;
  if (tid >= D)      // the dims beyond the head's are zeros, written once
    for (int j = 0; j < 2 * GR; ++j)
      rkw[j / GR][j % GR][0][padded(tid)] = rkw[j / GR][j % GR][1][padded(tid)] = rkw[j / GR][j % GR][2][padded(tid)] = 0.f;
  auto bring = [&](int first, int buf) {
    for (int j = 0; j < GR && first + j < t1; ++j) {
      const size_t t = first + j;
      if (tid < D) {
        copy_async4(&rkw[buf][j][0][padded(tid)], r + t * ld + head * D + tid);
        copy_async4(&rkw[buf][j][1][padded(tid)], k + t * ld + head * D + tid);
        copy_async4(&rkw[buf][j][2][padded(tid)], w + t * ldw + head * D + tid);
      }
      if (live && part == 0) copy_async4(&vs[buf][j][tid / P], v + t * ldv + head * V + col);
    }
    copy_async_commit();
  };
  bring(t0, 0);
  for (int first = t0; first < t1; first += GR) {
    const int buf = ((first - t0) / GR) & 1;
    if (first + GR < t1) {
      bring(first + GR, buf ^ 1);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const int n = min(GR, t1 - first);
    if (!AFTER) {
      for (int j = warp; j < n; j += P) {       // a token a warp: what the state has no part in
        float s = 0.f;
        for (int i = lane; i < DP; i += 32) s = fmaf(rkw[buf][j][0][padded(i)] * us[padded(i)], rkw[buf][j][1][padded(i)], s);
        s = warp_sum(s);
        if (lane == 0) ruk[j] = s;
      }
      __syncthreads();
    }
    for (int j = 0; j < n; ++j) {
      const float4* rs = (const float4*)(rkw[buf][j][0] + part * (SLICE + 4));
      const float4* ks = (const float4*)(rkw[buf][j][1] + part * (SLICE + 4));
      const float4* ws = (const float4*)(rkw[buf][j][2] + part * (SLICE + 4));
      const float vc = live ? vs[buf][j][tid / P] : 0.f;
      float sr = 0.f, sr2 = 0.f;
#pragma unroll
      for (int q = 0; q < SLICE / 4; ++q) {
        const float4 rv = rs[q], kv = ks[q], wv = ws[q];
        if (!AFTER) {
          sr = fmaf(S[4 * q], rv.x, sr); sr2 = fmaf(S[4 * q + 1], rv.y, sr2);
          sr = fmaf(S[4 * q + 2], rv.z, sr); sr2 = fmaf(S[4 * q + 3], rv.w, sr2);
        }
        S[4 * q] = fmaf(wv.x, S[4 * q], kv.x * vc);
        S[4 * q + 1] = fmaf(wv.y, S[4 * q + 1], kv.y * vc);
        S[4 * q + 2] = fmaf(wv.z, S[4 * q + 2], kv.z * vc);
        S[4 * q + 3] = fmaf(wv.w, S[4 * q + 3], kv.w * vc);
        if (AFTER) {
          sr = fmaf(S[4 * q], rv.x, sr); sr2 = fmaf(S[4 * q + 1], rv.y, sr2);
          sr = fmaf(S[4 * q + 2], rv.z, sr); sr2 = fmaf(S[4 * q + 3], rv.w, sr2);
        }
      }
      sr = lanes_sum<P>(sr + sr2);
      if (live && part == 0) y[(size_t)(first + j) * H * V + head * V + col] = (AFTER ? sr : fmaf(ruk[j], vc, sr)) * yscale;
    }
    __syncthreads();   // the group after next is brought into this buffer; ruk is written again
  }
  pdl_release_next();
  if (live) {
#pragma unroll
    for (int q = 0; q < SLICE / 4; ++q)
      Sg[((size_t)q * V + col) * P + part] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
  }
}

// r, k: rows of ld floats, w: rows of ldw floats, head h at h * D; v: rows of ldv floats, head h at h * V; bonus: [H, D],
// or null for the form whose read-out follows the write;
// state: [slots, H, gb_state_floats(D, V)] float32; y: [ntok, H * V].
// yscale multiplies every result (a factor on r, which the read-out is linear in).
GB_EXPORT int gb_wkv_scan_scaled(const float* r, const float* k, const float* w, long long ld, long long ldw, const float* v, long long ldv,
                                 const float* bonus, float* state, const int* cu, const int* seq_slot, float* y, int nseq, int H,
                                 int D, int V, float yscale, cudaStream_t stream) {
  if (nseq <= 0) return 0;
  if (H <= 0 || V <= 0 || D <= 0 || D > 8 * SLICE || ((uintptr_t)state & 15)) return GB_ERR_SIZE;
  dim3 grid(nseq, H, (V + 31) / 32);
#define GB_WKV(P, GR)                                                                                                       \
  if (bonus) launch_scan(wkv_scan_kernel<P, GR, false>, grid, 32 * P, stream, r, k, w, ld, ldw, v, ldv, bonus, state, cu, seq_slot, y, H, D, V, yscale); \
  else launch_scan(wkv_scan_kernel<P, GR, true>, grid, 32 * P, stream, r, k, w, ld, ldw, v, ldv, bonus, state, cu, seq_slot, y, H, D, V, yscale)
  switch (lanes_for(D)) {
    case 1: GB_WKV(1, 8); break;
    case 2: GB_WKV(2, 8); break;
    case 4: GB_WKV(4, 8); break;
    default: GB_WKV(8, 4);
  }
#undef GB_WKV
  return gb_launch_status();
}

GB_EXPORT int gb_wkv_scan(const float* r, const float* k, const float* w, long long ld, const float* v, long long ldv,
                          const float* bonus, float* state, const int* cu, const int* seq_slot, float* y, int nseq, int H, int D,
                          int V, cudaStream_t stream) {
  return gb_wkv_scan_scaled(r, k, w, ld, ld, v, ldv, bonus, state, cu, seq_slot, y, nseq, H, D, V, 1.0f, stream);
}
