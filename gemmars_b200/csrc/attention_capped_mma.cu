// bfloat16 attention with capped scores on the tensor cores (mma.sync), for prompts, parts of
// prompts and single positions alike: keys of GB_HEAD_DIM, values of GB_VALUE_DIM (compiled per
// pair of sizes), score = (q . k) * scale, then cap * tanh(score / cap) when cap > 0, a window when
// given (with `keep_first`, the keys 0..keep_first-1 are seen wherever the window stands), a sink
// per head when given (exp(sink[head]) joins the softmax's denominator, with no key and no value),
// and the output times sigmoid(gate) * out_scale when a gate is given.
//
// The arrangement is that of attention_prefill.cu: the 16 rows of an MMA are 16 consecutive
// tokens of one sequence for one query head, each row masked at its own position and window;
// keys (contiguous in the dims) and values (contiguous in the positions) feed the MMAs straight
// from the paged cache; a CTA covers 64 tokens of one sequence and up to two query heads that
// share a kv head.  A step of single tokens has a kernel of its own (below).  Scores,
// the cap, the softmax and the gate are float32; tanh is the hardware's approximation
// (tanh.approx.f32, relative error about 2^-11), which is below what bfloat16 operands leave.
#include "mma.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 128
#endif
#ifndef GB_VALUE_DIM
#define GB_VALUE_DIM GB_HEAD_DIM
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
constexpr int VD = GB_VALUE_DIM;
constexpr int KEYS = 32;
constexpr int TILE = 64;        // tokens per CTA
constexpr int MT = TILE / 16;   // row groups of 16 tokens
constexpr int RH = 2;           // query heads per CTA at most
constexpr int SPLIT = 8;        // warps that share a sequence's keys in a step of single tokens
constexpr float LOG2E = 1.4426950408889634f;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "key size must be a multiple of 16 up to 256");
static_assert(VD % 8 == 0 && VD >= 8 && VD <= 256, "value size must be a multiple of 8 up to 256");

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// grid (token tiles upper bound, kv heads * head chunks); block MT * heads_per_cta * 32.
__global__ void __launch_bounds__(MT * RH * 32)
attention_capped_mma_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                         const bf16* __restrict__ kcache, const bf16* __restrict__ vcache, PagedKV kv,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_slot, int n_seqs, int nh, int window, int keep_first,
                         const float* __restrict__ sink, int heads_per_cta, float scale,
                         float cap, const bf16* __restrict__ gate, long long gate_stride, float out_scale) {
  pdl_release_next();
  pdl_wait_prior();
  // ---- which sequence and which 64-token tile of it
  int b = 0, tile = blockIdx.x;
  for (; b < n_seqs; ++b) {
    const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + TILE - 1) / TILE;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= n_seqs) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int mt = warp % MT, hr = warp / MT;
  const int rep = nh / kv.num_kv_heads;
  const int chunks = (rep + heads_per_cta - 1) / heads_per_cta;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int hl = chunk * heads_per_cta + hr;          // head within the kv group
  if (hl >= rep) return;
  const int head = kvh * rep + hl;
  const int seq_len = cu_seqlens[b + 1] - cu_seqlens[b];
  const int first = tile * TILE + mt * 16;            // first token of this warp within the sequence's step
  if (first >= seq_len) return;
  const int slot = seq_slot[b], start = seq_start[b];
  const int tok0 = cu_seqlens[b] + first;
  const bool v0 = first + g < seq_len, v1 = first + g + 8 < seq_len;
  const int pos0 = v0 ? start + first + g : -1, pos1 = v1 ? start + first + g + 8 : -1;   // -1: no key passes
  const int last = start + min(first + 15, seq_len - 1);                                    // last position of the warp
  const int lo_first = window > 0 ? max(0, start + first + 1 - window) : 0;
  const int lo0 = window > 0 ? max(0, pos0 + 1 - window) : 0, lo1 = window > 0 ? max(0, pos1 + 1 - window) : 0;

  constexpr int KB = HD / 32, TAIL = HD % 32;
  uint32_t qa[KB + 1][4], qb[KB + 1][4];
  {
    const bf16* q0 = q + (size_t)(tok0 + g) * q_stride + (size_t)head * HD;
    const bf16* q1 = q0 + 8 * q_stride;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      uint4 a = v0 ? *(const uint4*)(q0 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qa[kb][0] = a.x; qa[kb][1] = a.y; qa[kb][2] = a.z; qa[kb][3] = a.w;
      uint4 bb = v1 ? *(const uint4*)(q1 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qb[kb][0] = bb.x; qb[kb][1] = bb.y; qb[kb][2] = bb.z; qb[kb][3] = bb.w;
    }
    if (TAIL) {
      uint2 a = v0 ? *(const uint2*)(q0 + KB * 32 + c * 4) : make_uint2(0, 0);
      qa[KB][0] = a.x; qa[KB][1] = a.y;
      uint2 bb = v1 ? *(const uint2*)(q1 + KB * 32 + c * 4) : make_uint2(0, 0);
      qb[KB][0] = bb.x; qb[KB][1] = bb.y;
    }
  }

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[VD / 8][4];
#pragma unroll
  for (int d = 0; d < VD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f, cap2 = cap * LOG2E, scale2 = scale * LOG2E;
  // blocks of 32 keys: first those of the kept keys that lie below the window's first block, then the window's
  const int win_blk = lo_first / KEYS, kept_blks = min((keep_first + KEYS - 1) / KEYS, win_blk);
  const int n_blks = kept_blks + last / KEYS - win_blk + 1;
  for (int it = 0; it < n_blks; ++it) {
    const int key0 = (it < kept_blks ? it : win_blk + it - kept_blks) * KEYS;
    const int page = kv.page_table[(size_t)slot * kv.table_width + (key0 / kv.page_size) % kv.table_width];
    const size_t page_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * HD;
    const size_t value_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * VD;
    const int in_page = key0 % kv.page_size;
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const bf16* krow = kcache + page_base + (size_t)(in_page + 8 * (g >> 1) + 2 * j + (g & 1)) * HD;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        const uint4 k4 = *(const uint4*)(krow + kb * 32 + c * 8);
        mma16816(s[j], qa[kb][0], qb[kb][0], qa[kb][1], qb[kb][1], k4.x, k4.y);
        mma16816(s[j], qa[kb][2], qb[kb][2], qa[kb][3], qb[kb][3], k4.z, k4.w);
      }
      if (TAIL) {
        const uint2 k2 = *(const uint2*)(krow + KB * 32 + c * 4);
        mma16816(s[j], qa[KB][0], qb[KB][0], qa[KB][1], qb[KB][1], k2.x, k2.y);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * c + 2 * j + e;
        // in log2 units: cap * tanh(score * scale / cap) * log2(e), or score * scale * log2(e)
        const float a0 = cap > 0.f ? cap2 * tanh_fast(s[j][e] * scale * inv_cap) : s[j][e] * scale2;
        const float a1 = cap > 0.f ? cap2 * tanh_fast(s[j][2 + e] * scale * inv_cap) : s[j][2 + e] * scale2;
        s[j][e] = ((key >= lo0 || key < keep_first) && key <= pos0) ? a0 : -INFINITY;
        s[j][2 + e] = ((key >= lo1 || key < keep_first) && key <= pos1) ? a1 : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    const float n0 = fmaxf(m0, quad_max(mx0)), n1 = fmaxf(m1, quad_max(mx1));
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float alpha0 = exp2f(m0 - u0), alpha1 = exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    uint32_t p[4][2];
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = exp2f(s[j][0] - u0), bb = exp2f(s[j][1] - u0);
      const float cc = exp2f(s[j][2] - u1), d = exp2f(s[j][3] - u1);
      sum0 += a + bb;
      sum1 += cc + d;
      p[j][0] = pack_bf16(a, bb);
      p[j][1] = pack_bf16(cc, d);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
    const bf16* vbase = vcache + value_base + in_page + 8 * c;
#pragma unroll
    for (int d = 0; d < VD / 8; ++d) {
      const uint4 v4 = *(const uint4*)(vbase + (size_t)(d * 8 + g) * kv.page_size);
      o[d][0] *= alpha0; o[d][1] *= alpha0; o[d][2] *= alpha1; o[d][3] *= alpha1;
      mma16816(o[d], p[0][0], p[0][1], p[1][0], p[1][1], v4.x, v4.y);
      mma16816(o[d], p[2][0], p[2][1], p[3][0], p[3][1], v4.z, v4.w);
    }
  }
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  float keep0 = 1.f, keep1 = 1.f;       // what the sink leaves of the keys' share
  if (sink) {
    const float s2 = sink[head] * LOG2E, n0 = fmaxf(m0, s2), n1 = fmaxf(m1, s2);
    keep0 = m0 == -INFINITY ? 0.f : exp2f(m0 - n0);
    keep1 = m1 == -INFINITY ? 0.f : exp2f(m1 - n1);
    l0 = l0 * keep0 + exp2f(s2 - n0);
    l1 = l1 * keep1 + exp2f(s2 - n1);
  }
  if (v0) {
    const float inv = out_scale * keep0 / l0;
    bf16* dst = out + (size_t)(tok0 + g) * out_stride + (size_t)head * VD + 2 * c;
    const bf16* gt = gate ? gate + (size_t)(tok0 + g) * gate_stride + (size_t)head * VD + 2 * c : nullptr;
#pragma unroll
    for (int d = 0; d < VD / 8; ++d) {
      float a = o[d][0] * inv, bb = o[d][1] * inv;
      if (gt) {
        const float2 z = __bfloat1622float2(*(const __nv_bfloat162*)(gt + d * 8));
        a *= 1.0f / (1.0f + __expf(-z.x));
        bb *= 1.0f / (1.0f + __expf(-z.y));
      }
      *(uint32_t*)(dst + d * 8) = pack_bf16(a, bb);
    }
  }
  if (v1) {
    const float inv = out_scale * keep1 / l1;
    bf16* dst = out + (size_t)(tok0 + g + 8) * out_stride + (size_t)head * VD + 2 * c;
    const bf16* gt = gate ? gate + (size_t)(tok0 + g + 8) * gate_stride + (size_t)head * VD + 2 * c : nullptr;
#pragma unroll
    for (int d = 0; d < VD / 8; ++d) {
      float a = o[d][2] * inv, bb = o[d][3] * inv;
      if (gt) {
        const float2 z = __bfloat1622float2(*(const __nv_bfloat162*)(gt + d * 8));
        a *= 1.0f / (1.0f + __expf(-z.x));
        bb *= 1.0f / (1.0f + __expf(-z.y));
      }
      *(uint32_t*)(dst + d * 8) = pack_bf16(a, bb);
    }
  }
}

// A step of single tokens.  The 16 rows of an MMA are the query heads that share a kv head (in
// chunks of 16), all at the sequence's one new position, so a key or value is read once for all
// of them; the SPLIT warps of a CTA take every SPLIT-th block of 32 keys each, and their parts
// (maximum, sum, weighted values per row) meet in shared memory, added in warp order.
// grid (sequences, kv heads * chunks of 16 heads); block SPLIT * 32.
__global__ void __launch_bounds__(SPLIT * 32)
attention_capped_single_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                         const bf16* __restrict__ kcache, const bf16* __restrict__ vcache, PagedKV kv,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_slot, int n_seqs, int nh, int window, int keep_first,
                         const float* __restrict__ sink, float scale,
                         float cap, const bf16* __restrict__ gate, long long gate_stride, float out_scale) {
  pdl_release_next();
  pdl_wait_prior();
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rep = nh / kv.num_kv_heads;
  const int chunks = (rep + 15) / 16;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int head_base = kvh * rep + chunk * 16;       // row r of the MMA is query head head_base + r
  const int rows = min(16, rep - chunk * 16);
  const int slot = seq_slot[b], start = seq_start[b];
  const int tok0 = cu_seqlens[b];
  const bool v0 = g < rows, v1 = g + 8 < rows;
  const int pos0 = v0 ? start : -1, pos1 = v1 ? start : -1;   // -1: no key passes
  const int last = start;
  const int lo_first = window > 0 ? max(0, start + 1 - window) : 0;
  const int lo0 = lo_first, lo1 = lo_first;

  constexpr int KB = HD / 32, TAIL = HD % 32;
  uint32_t qa[KB + 1][4], qb[KB + 1][4];
  {
    const bf16* q0 = q + (size_t)tok0 * q_stride + (size_t)(head_base + g) * HD;
    const bf16* q1 = q0 + 8 * HD;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      uint4 a = v0 ? *(const uint4*)(q0 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qa[kb][0] = a.x; qa[kb][1] = a.y; qa[kb][2] = a.z; qa[kb][3] = a.w;
      uint4 bb = v1 ? *(const uint4*)(q1 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qb[kb][0] = bb.x; qb[kb][1] = bb.y; qb[kb][2] = bb.z; qb[kb][3] = bb.w;
    }
    if (TAIL) {
      uint2 a = v0 ? *(const uint2*)(q0 + KB * 32 + c * 4) : make_uint2(0, 0);
      qa[KB][0] = a.x; qa[KB][1] = a.y;
      uint2 bb = v1 ? *(const uint2*)(q1 + KB * 32 + c * 4) : make_uint2(0, 0);
      qb[KB][0] = bb.x; qb[KB][1] = bb.y;
    }
  }

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[VD / 8][4];
#pragma unroll
  for (int d = 0; d < VD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f, cap2 = cap * LOG2E, scale2 = scale * LOG2E;
  const int win_blk = lo_first / KEYS, kept_blks = min((keep_first + KEYS - 1) / KEYS, win_blk);
  const int n_blks = kept_blks + last / KEYS - win_blk + 1;
  for (int it = warp; it < n_blks; it += SPLIT) {
    const int key0 = (it < kept_blks ? it : win_blk + it - kept_blks) * KEYS;
    const int page = kv.page_table[(size_t)slot * kv.table_width + (key0 / kv.page_size) % kv.table_width];
    const size_t page_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * HD;
    const size_t value_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * VD;
    const int in_page = key0 % kv.page_size;
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const bf16* krow = kcache + page_base + (size_t)(in_page + 8 * (g >> 1) + 2 * j + (g & 1)) * HD;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        const uint4 k4 = *(const uint4*)(krow + kb * 32 + c * 8);
        mma16816(s[j], qa[kb][0], qb[kb][0], qa[kb][1], qb[kb][1], k4.x, k4.y);
        mma16816(s[j], qa[kb][2], qb[kb][2], qa[kb][3], qb[kb][3], k4.z, k4.w);
      }
      if (TAIL) {
        const uint2 k2 = *(const uint2*)(krow + KB * 32 + c * 4);
        mma16816(s[j], qa[KB][0], qb[KB][0], qa[KB][1], qb[KB][1], k2.x, k2.y);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * c + 2 * j + e;
        // in log2 units: cap * tanh(score * scale / cap) * log2(e), or score * scale * log2(e)
        const float a0 = cap > 0.f ? cap2 * tanh_fast(s[j][e] * scale * inv_cap) : s[j][e] * scale2;
        const float a1 = cap > 0.f ? cap2 * tanh_fast(s[j][2 + e] * scale * inv_cap) : s[j][2 + e] * scale2;
        s[j][e] = ((key >= lo0 || key < keep_first) && key <= pos0) ? a0 : -INFINITY;
        s[j][2 + e] = ((key >= lo1 || key < keep_first) && key <= pos1) ? a1 : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    const float n0 = fmaxf(m0, quad_max(mx0)), n1 = fmaxf(m1, quad_max(mx1));
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float alpha0 = exp2f(m0 - u0), alpha1 = exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    uint32_t p[4][2];
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = exp2f(s[j][0] - u0), bb = exp2f(s[j][1] - u0);
      const float cc = exp2f(s[j][2] - u1), d = exp2f(s[j][3] - u1);
      sum0 += a + bb;
      sum1 += cc + d;
      p[j][0] = pack_bf16(a, bb);
      p[j][1] = pack_bf16(cc, d);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
    const bf16* vbase = vcache + value_base + in_page + 8 * c;
#pragma unroll
    for (int d = 0; d < VD / 8; ++d) {
      const uint4 v4 = *(const uint4*)(vbase + (size_t)(d * 8 + g) * kv.page_size);
      o[d][0] *= alpha0; o[d][1] *= alpha0; o[d][2] *= alpha1; o[d][3] *= alpha1;
      mma16816(o[d], p[0][0], p[0][1], p[1][0], p[1][1], v4.x, v4.y);
      mma16816(o[d], p[2][0], p[2][1], p[3][0], p[3][1], v4.z, v4.w);
    }
  }
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  extern __shared__ float parts[];            // [SPLIT][16] maxima, [SPLIT][16] sums, [SPLIT][16][VD] weighted values
  float* pm = parts;
  float* pl = pm + SPLIT * 16;
  float* po = pl + SPLIT * 16;
  if (c == 0) {
    pm[warp * 16 + g] = m0; pl[warp * 16 + g] = l0;
    pm[warp * 16 + g + 8] = m1; pl[warp * 16 + g + 8] = l1;
  }
#pragma unroll
  for (int d = 0; d < VD / 8; ++d) {
    *(float2*)(po + (size_t)(warp * 16 + g) * VD + d * 8 + 2 * c) = make_float2(o[d][0], o[d][1]);
    *(float2*)(po + (size_t)(warp * 16 + g + 8) * VD + d * 8 + 2 * c) = make_float2(o[d][2], o[d][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * VD; idx += SPLIT * 32) {
    const int row = idx / VD, col = idx - row * VD;
    const float s2 = sink ? sink[head_base + row] * LOG2E : -INFINITY;
    float top = s2;
#pragma unroll
    for (int w = 0; w < SPLIT; ++w) top = fmaxf(top, pm[w * 16 + row]);
    float total = sink ? exp2f(s2 - top) : 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < SPLIT; ++w) {
      const float m = pm[w * 16 + row];
      const float wt = m == -INFINITY ? 0.f : exp2f(m - top);
      total = fmaf(wt, pl[w * 16 + row], total);
      acc = fmaf(wt, po[(size_t)(w * 16 + row) * VD + col], acc);
    }
    float a = acc * out_scale / total;
    const size_t at = (size_t)(head_base + row) * VD + col;
    if (gate) a *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(size_t)tok0 * gate_stride + at])));
    out[(size_t)tok0 * out_stride + at] = __float2bfloat16_rn(a);
  }
}

}  // namespace

// q: [ntok, nh * HD], out: [ntok, nh * VD] bfloat16, tokens of all sequences packed (cu_seqlens:
// [n_seqs + 1]); seq_start: cache length of each sequence before this step; the cache already holds
// this step's keys and values.  q rows must be 16-byte aligned, out and gate rows 4-byte aligned.
GB_EXPORT int gb_attention_capped_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, const int* page_table, int table_width,
                                      int page_size, int nkv, int hd, int vd, const int* cu_seqlens, const int* seq_start,
                                      const int* seq_slot, int n_seqs, int ntok, int nh, int window, int keep_first,
                                      const float* sink, float scale, float cap, const void* gate, long long gate_stride, float out_scale, int single, cudaStream_t stream) {
  if (ntok <= 0 || n_seqs <= 0) return 0;
  if (hd != HD || vd != VD || nkv <= 0 || nh % nkv || page_size % KEYS || keep_first < 0) return GB_ERR_SIZE;
  if (window <= 0) keep_first = 0;      // every key is seen already
  if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)out & 3) || (out_stride % 2) || ((uintptr_t)kcache & 15) ||
      ((uintptr_t)vcache & 15) || ((uintptr_t)gate & 3) || (gate_stride % 2))
    return GB_ERR_SIZE;
  PagedKV kv{page_table, table_width, page_size, nkv, hd};
  const int rep = nh / nkv;
  const int heads_per_cta = rep < RH ? rep : RH;
  const int chunks = (rep + heads_per_cta - 1) / heads_per_cta;
  if (single) {
    // every sequence brings one token (ntok == n_seqs)
    if (ntok != n_seqs) return GB_ERR_ARG;
    const size_t smem = (size_t)SPLIT * 16 * (VD + 2) * sizeof(float);
    static bool raised = false;
    if (!raised) {
      cudaFuncSetAttribute(attention_capped_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      raised = true;
    }
    const dim3 sgrid(n_seqs, nkv * ((rep + 15) / 16));
    if ((size_t)sgrid.x * sgrid.y > 2 * 148) {
      gb_launch(attention_capped_single_kernel, sgrid, SPLIT * 32, smem, stream,
          (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, kv, cu_seqlens,
          seq_start, seq_slot, n_seqs, nh, window, keep_first, sink, scale, cap, (const bf16*)gate, gate_stride, out_scale);
    } else {
      // few CTAs: started only when the kernel before has ended, so that they spread one to an SM instead of
      // sharing the few SMs that had room while that kernel ran
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = sgrid;
      cfg.blockDim = dim3(SPLIT * 32);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchKernelEx(&cfg, attention_capped_single_kernel,
          (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, kv, cu_seqlens,
          seq_start, seq_slot, n_seqs, nh, window, keep_first, sink, scale, cap, (const bf16*)gate, gate_stride, out_scale);
    }
    return gb_launch_status();
  }
  dim3 grid((ntok + TILE - 1) / TILE + n_seqs, nkv * chunks);
  gb_launch(attention_capped_mma_kernel, grid, MT * heads_per_cta * 32, 0, stream,
      (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, kv, cu_seqlens,
      seq_start, seq_slot, n_seqs, nh, window, keep_first, sink, heads_per_cta, scale, cap, (const bf16*)gate, gate_stride, out_scale);
  return gb_launch_status();
}
