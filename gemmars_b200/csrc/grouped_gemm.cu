// Grouped bfloat16 products on the tensor cores: many products  C_g = A_g W_g^T  of unequal row
// counts in one launch, the row counts known on the device alone.  Two users:
//
//  * the experts of a routed feed-forward for more than a few tokens: group = expert, the rows of
//    a group are the (token, slot) entries routed to it (gb_moe_sort orders them), A rows are
//    gathered by token, W_g is the expert's matrix.  The gate/up product applies the experts'
//    activation in its epilogue (the tile interleaves 8 gate rows with the 8 up rows of the same
//    features, so a thread holds both); the down product scales each row by its routing weight and
//    leaves float32 rows that gb_moe_combine adds into the residual in slot order.  (Prompt steps
//    run the same two products on the tcgen05 kernel of gemm_tc.cu instead, from a copy of the
//    activations in a padded order: gb_moe_sort_padded, gb_moe_permute.)
//  * the per-head products of latent attention: group = head, every group has all the tokens,
//    A and C rows are a token's slice of a wider row, with an optional scale per (token, head).
//
// A CTA of 8 warps computes a tile of 128 rows x 128 columns (mma.sync m16n8k16, float32
// accumulation), operands staged in shared memory by cp.async three blocks of 64 deep.  A CTA
// finds its group and row tile by walking the groups' offsets, so nothing comes back to the host
// and the launches can be captured.
#include "mma.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3, LDS = BK + 8;
constexpr int CPR = BK / 8;          // 16-byte pieces of a row of a block
constexpr int RPT = BM * CPR / 256;  // rows a thread brings in
enum { MODE_PLAIN = 0, MODE_GATED = 1 };

struct GroupedArgs {
  const bf16* a; long long lda; long long a_gstride;
  const int* a_rows; int a_div;              // A row of entry i: a_rows ? a_rows[i] / a_div : i
  const bf16* w; long long w_gstride;        // W_g = w + g * w_gstride, [N (2N gated), K] row-major
  void* c; long long ldc; long long c_gstride;
  const float* scale; const int* scale_rows; long long s_rstride; long long s_gstride;
  const int* offsets;                        // [groups + 1], or null: every group has `rows` rows
  int groups, rows, N, K;
  float limit, alpha, shift;                 // gated: g = min(g, limit), u = clamp(u, +-limit), g * sigmoid(alpha g) * (u + shift)
  int act;                                   // plain mode: 1 = the exact (erf) GELU of every result before the scale
};
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ void cp_async16_or_zero(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;          // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

__device__ __forceinline__ void store2(float* p, float x, float y) { *(float2*)p = make_float2(x, y); }
__device__ __forceinline__ void store2(bf16* p, float x, float y) { *(uint32_t*)p = pack_bf16(x, y); }

template <int MODE, typename TO>
__global__ void __launch_bounds__(256, 2) grouped_gemm_kernel(GroupedArgs p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_release_next();
  pdl_wait_prior();
  bf16* As = (bf16*)smem_raw;                          // [STAGES][BM][LDS]
  bf16* Ws = As + STAGES * BM * LDS;                   // [STAGES][BN][LDS]
  // ---- group and row tile
  int g, mt, row0, cnt;
  if (p.offsets == nullptr) {
    const int tpg = (p.rows + BM - 1) / BM;
    g = blockIdx.x / tpg; mt = blockIdx.x % tpg; row0 = 0; cnt = p.rows;
    if (g >= p.groups) return;
  } else {
    int left = blockIdx.x;
    for (g = 0; g < p.groups; ++g) {
      row0 = p.offsets[g];
      cnt = p.offsets[g + 1] - row0;
      const int tiles = (cnt + BM - 1) / BM;
      if (left < tiles) break;
      left -= tiles;
    }
    if (g >= p.groups) return;
    mt = left;
  }
  const int n0 = blockIdx.y * (MODE == MODE_GATED ? BN / 2 : BN);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wn = warp & 3;             // 2 x 4 warps, 64 rows x 32 columns each
  // ---- the A rows and W rows this thread brings in, every block of K
  const int ch = tid % CPR;
  const bf16* a_src[RPT];
  const bf16* w_src[RPT];
  bool a_ok[RPT], w_ok[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = tid / CPR + (256 / CPR) * i;
    const int lr = mt * BM + r;
    a_ok[i] = lr < cnt;
    long long arow = 0;
    if (a_ok[i]) arow = p.a_rows ? p.a_rows[row0 + lr] / p.a_div : row0 + lr;
    a_src[i] = p.a + arow * p.lda + (long long)g * p.a_gstride + ch * 8;
    int wrow;
    if (MODE == MODE_GATED) {
      const int f = n0 + (r >> 4) * 8 + (r & 7);
      w_ok[i] = f < p.N;
      wrow = (r & 8) ? p.N + f : f;
    } else {
      wrow = n0 + r;
      w_ok[i] = wrow < p.N;
    }
    w_src[i] = p.w + (long long)g * p.w_gstride + (long long)(w_ok[i] ? wrow : 0) * p.K + ch * 8;
  }
  const int kblocks = (p.K + BK - 1) / BK;
  auto load = [&](int kb, int stage) {
    const bool k_ok = kb * BK + ch * 8 < p.K;          // K is a multiple of 8: a piece is whole or absent
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = tid / CPR + (256 / CPR) * i;
      cp_async16_or_zero(As + ((size_t)stage * BM + r) * LDS + ch * 8, a_src[i] + (size_t)kb * BK, a_ok[i] && k_ok);
      cp_async16_or_zero(Ws + ((size_t)stage * BN + r) * LDS + ch * 8, w_src[i] + (size_t)kb * BK, w_ok[i] && k_ok);
    }
  };
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < kblocks) load(s, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const int a_off = (wm * 64 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + 8 * (lane >> 4);
  const int w_off = (wn * 32 + (lane & 7) + 8 * (lane >> 4)) * LDS + 8 * ((lane >> 3) & 1);
  for (int kb = 0; kb < kblocks; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    if (kb + STAGES - 1 < kblocks) load(kb + STAGES - 1, (kb + STAGES - 1) % STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* at = As + (size_t)(kb % STAGES) * BM * LDS + a_off;
    const bf16* wt = Ws + (size_t)(kb % STAGES) * BN * LDS + w_off;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t af[4][4], bfr[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ldsm4(af[i], at + i * 16 * LDS + ks * 16);
#pragma unroll
      for (int j = 0; j < 2; ++j) ldsm4(bfr[j], wt + j * 16 * LDS + ks * 16);   // columns 16j..16j+7: regs 0,1; 16j+8..: regs 2,3
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma16816(acc[i][j], af[i][0], af[i][1], af[i][2], af[i][3], bfr[j >> 1][2 * (j & 1)], bfr[j >> 1][2 * (j & 1) + 1]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // ---- epilogue
  const int gq = lane >> 2, cq = lane & 3;
  TO* cbase = (TO*)p.c + (long long)g * p.c_gstride;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int lr = mt * BM + wm * 64 + i * 16 + gq + 8 * half;
      if (lr >= cnt) continue;
      const long long crow = row0 + lr;
      float sc = 1.f;
      if (p.scale) {
        const long long srow = p.scale_rows ? p.scale_rows[crow] : crow;
        sc = p.scale[srow * p.s_rstride + (long long)g * p.s_gstride];
      }
      TO* dst = cbase + crow * p.ldc;
      if (MODE == MODE_GATED) {
#pragma unroll
        for (int j = 0; j < 4; j += 2)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int f = n0 + (wn * 2 + (j >> 1)) * 8 + 2 * cq + e;
            if (f >= p.N) continue;
            const float gt = fminf(acc[i][j][2 * half + e], p.limit);
            const float up = fminf(fmaxf(acc[i][j + 1][2 * half + e], -p.limit), p.limit);
            dst[f] = from_f32<TO>(gt / (1.0f + expf(-p.alpha * gt)) * (up + p.shift) * sc);
          }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = n0 + wn * 32 + j * 8 + 2 * cq;
          float x = acc[i][j][2 * half], y = acc[i][j][2 * half + 1];
          if (p.act == 1) { x = gelu_erf_f(x); y = gelu_erf_f(y); }
          x *= sc; y *= sc;
          if (col + 1 < p.N && ((uintptr_t)(dst + col) & (2 * sizeof(TO) - 1)) == 0) {
            store2(dst + col, x, y);
          } else {
            if (col < p.N) dst[col] = from_f32<TO>(x);
            if (col + 1 < p.N) dst[col + 1] = from_f32<TO>(y);
          }
        }
      }
    }
}

// One block: orders the (token, slot) entries of a step by expert.  offsets[e]..offsets[e+1] are
// expert e's places in `perm` (entry = token * top + slot); place[entry] is where the entry went.
// The order inside an expert is whatever the atomics give: every row is computed by itself, and
// the sums over a token's slots are taken in slot order afterwards.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int entries, int E,
                                                        int* __restrict__ offsets, int* __restrict__ perm,
                                                        int* __restrict__ place) {
  extern __shared__ int counts[];   // [E] counts, then [E] running starts
  pdl_release_next();
  pdl_wait_prior();
  int* starts = counts + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { offsets[e] = acc; starts[e] = acc; acc += counts[e]; }
    offsets[E] = acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int at = atomicAdd(&starts[idx[i]], 1);
    perm[at] = i;
    place[i] = at;
  }
}

// As moe_sort_kernel, for the tcgen05 product that wants every expert's rows to start at a multiple
// of `bn` rows: place[entry] is the entry's row in that padded order, row_entry[row] the entry of a
// row (-1: padding), tile_expert[row / bn] the expert a tile of bn rows belongs to (-1: none).
__global__ void __launch_bounds__(1024) moe_sort_padded_kernel(const int* __restrict__ idx, int entries, int E, int bn,
                                                               int rows, int* __restrict__ tile_expert,
                                                               int* __restrict__ place, int* __restrict__ row_entry) {
  extern __shared__ int counts[];   // [E] counts, then [E] running starts
  pdl_release_next();
  pdl_wait_prior();
  int* starts = counts + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) row_entry[r] = -1;
  for (int t = threadIdx.x; t < rows / bn; t += blockDim.x) tile_expert[t] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      starts[e] = acc;
      const int tiles = (counts[e] + bn - 1) / bn;
      for (int t = 0; t < tiles; ++t) tile_expert[acc / bn + t] = e;
      acc += tiles * bn;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int at = atomicAdd(&starts[idx[i]], 1);
    place[i] = at;
    row_entry[at] = i;
  }
}

// The activations in the padded order: row r = h[token of its entry], zeros for padding inside a used
// tile (tiles that no expert uses are never read); scale[r] = the entry's routing weight.
__global__ void __launch_bounds__(128) moe_permute_kernel(const bf16* __restrict__ h, long long ldh,
                                                          const int* __restrict__ row_entry, const int* __restrict__ tile_expert,
                                                          const float* __restrict__ wts, bf16* __restrict__ xp,
                                                          float* __restrict__ scale, int width, int top, int bn) {
  pdl_release_next();
  pdl_wait_prior();
  const int r = blockIdx.x;
  if (tile_expert[r / bn] < 0) return;
  const int e = row_entry[r];
  uint4* dst = (uint4*)(xp + (size_t)r * width);
  if (e < 0) {
    for (int i = threadIdx.x; i < width / 8; i += 128) dst[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) scale[r] = 0.f;
    return;
  }
  const uint4* src = (const uint4*)(h + (size_t)(e / top) * ldh);
  for (int i = threadIdx.x; i < width / 8; i += 128) dst[i] = src[i];
  if (threadIdx.x == 0) scale[r] = wts[e];
}

// residual[t] += sum over the token's slots, in slot order, of the rows the down product left
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ place,
                                                          float* __restrict__ residual, long long ldr, int width, int top) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < width; n += 256) {
    float total = 0.f;
    for (int k = 0; k < top; ++k) total += rows[(size_t)place[(size_t)t * top + k] * width + n];
    residual[(size_t)t * ldr + n] += total;
  }
}

// y[t, f] = act(gu[t, f], gu[t, F + f]) * scale[t]: the activation of a dense (shared) expert
__global__ void __launch_bounds__(256) gated_act_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y,
                                                        const float* __restrict__ scale, int F, float limit, float alpha,
                                                        float shift) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const float sc = scale ? scale[t] : 1.f;
  for (int f = threadIdx.x; f < F; f += 256) {
    const float gt = fminf(__bfloat162float(gu[(size_t)t * 2 * F + f]), limit);
    const float up = fminf(fmaxf(__bfloat162float(gu[(size_t)t * 2 * F + F + f]), -limit), limit);
    y[(size_t)t * F + f] = __float2bfloat16_rn(gt / (1.0f + expf(-alpha * gt)) * (up + shift) * sc);
  }
}

template <int MODE, typename TO>
int launch_grouped(const GroupedArgs& p, int row_tiles, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (BM + BN) * LDS * sizeof(bf16);
  static bool allowed = false;
  if (!allowed) {
    if (cudaFuncSetAttribute(grouped_gemm_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return GB_ERR_SIZE;
    allowed = true;
  }
  const int per = MODE == MODE_GATED ? BN / 2 : BN;
  dim3 grid(row_tiles, (p.N + per - 1) / per);
  gb_launch(grouped_gemm_kernel<MODE, TO>, grid, dim3(256), smem, stream, p);
  return gb_launch_status();
}

}  // namespace

// The general form; see GroupedArgs.  out_f32: C is float32 (else bfloat16); gated 1: W_g has 2N rows
// and C = act(gate, up) in bfloat16; gated 2: W_g has N rows and C = gelu(A W_g^T) (erf form).  max_rows: an upper bound of the rows over all groups (the
// grid is sized by it when the counts live on the device).
GB_EXPORT int gb_grouped_gemm(const void* a, long long lda, long long a_gstride, const int* a_rows, int a_div,
                              const void* w, long long w_gstride, void* c, long long ldc, long long c_gstride,
                              const float* scale, const int* scale_rows, long long s_rstride, long long s_gstride,
                              const int* offsets, int groups, int rows, int max_rows, int N, int K, int gated, int out_f32,
                              float limit, float alpha, float shift, cudaStream_t stream) {
  if (groups <= 0 || N <= 0 || max_rows <= 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || a_gstride % 8 || w_gstride % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return GB_ERR_SIZE;
  if (gated == 1 && out_f32) return GB_ERR_DTYPE;
  if (gated < 0 || gated > 2) return GB_ERR_ARG;
  GroupedArgs p{(const bf16*)a, lda, a_gstride, a_rows, a_div > 0 ? a_div : 1, (const bf16*)w, w_gstride, c, ldc, c_gstride,
                scale, scale_rows, s_rstride, s_gstride, offsets, groups, rows, N, K, limit, alpha, shift, gated == 2 ? 1 : 0};
  const int row_tiles = offsets ? (max_rows + BM - 1) / BM + groups : groups * ((rows + BM - 1) / BM);
  if (gated == 1) return launch_grouped<MODE_GATED, bf16>(p, row_tiles, stream);
  if (out_f32) return launch_grouped<MODE_PLAIN, float>(p, row_tiles, stream);
  return launch_grouped<MODE_PLAIN, bf16>(p, row_tiles, stream);
}

GB_EXPORT int gb_moe_sort(const int* idx, int entries, int E, int* offsets, int* perm, int* place, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (E <= 0 || E > 4096) return GB_ERR_SIZE;
  gb_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, idx, entries, E, offsets, perm, place);
  return gb_launch_status();
}

GB_EXPORT int gb_moe_sort_padded(const int* idx, int entries, int E, int bn, int rows, int* tile_expert, int* place,
                                 int* row_entry, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (E <= 0 || E > 4096 || bn <= 0 || rows % bn || rows < entries + E * (bn - 1)) return GB_ERR_SIZE;
  gb_launch(moe_sort_padded_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, idx, entries, E, bn, rows,
            tile_expert, place, row_entry);
  return gb_launch_status();
}

// h: [ntok, width] bfloat16 rows ldh apart (width % 8 == 0, 16-byte aligned rows); xp: [rows, width]
GB_EXPORT int gb_moe_permute(const void* h, long long ldh, const int* row_entry, const int* tile_expert, const float* wts,
                             void* xp, float* scale, int rows, int width, int top, int bn, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width % 8 || ldh % 8 || ((uintptr_t)h & 15) || ((uintptr_t)xp & 15)) return GB_ERR_SIZE;
  gb_launch(moe_permute_kernel, dim3(rows), dim3(128), 0, stream, (const bf16*)h, ldh, row_entry, tile_expert, wts, (bf16*)xp,
            scale, width, top, bn);
  return gb_launch_status();
}

GB_EXPORT int gb_moe_combine(const float* rows, const int* place, float* residual, long long ldr, int ntok, int width, int top,
                             cudaStream_t stream) {
  if (ntok <= 0) return 0;
  gb_launch(moe_combine_kernel, dim3(ntok), dim3(256), 0, stream, rows, place, residual, ldr, width, top);
  return gb_launch_status();
}

GB_EXPORT int gb_gated_act(const void* gu, void* y, const float* scale, int ntok, int F, float limit, float alpha, float shift,
                           cudaStream_t stream) {
  if (ntok <= 0 || F <= 0) return 0;
  gb_launch(gated_act_kernel, dim3(ntok), dim3(256), 0, stream, (const bf16*)gu, (bf16*)y, scale, F, limit, alpha, shift);
  return gb_launch_status();
}
