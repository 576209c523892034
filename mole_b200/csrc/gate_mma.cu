// bf16 backward products of the gate on the warp-level tensor-core path:
//
//   dispatch_bwd_mma_kernel   dx[t, :] = sum_j kept * ddisp[row(t, j), :] + dlogits[t, :] @ Wg
//   gate_wgrad_mma_kernel     dWg[e, :] += sum_t dlogits[t, e] * x[t, :]
//
// Both contain a product with one tiny dimension (E <= 256 experts).  On CUDA cores they were
// FMA-bound at 5-8 % of the HBM rate they should run at; a tcgen05 pipeline does not pay for a
// 64-wide contraction.  mma.sync m16n8k16 with fp32 accumulation does.  dlogits is fp32: it
// enters the bf16 MMA as hi + lo (two bf16 terms, two MMAs), which keeps 16 mantissa bits; the
// other operand (Wg, x) is bf16 already.  The fp32 layer keeps the CUDA-core kernels.
#include "common.cuh"

namespace mole {

__device__ __forceinline__ void ldsm_x4(const void* p, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(const void* p, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

constexpr int kGmTok = 64;       // tokens per MMA tile
constexpr int kGmCols = 128;     // columns per block
constexpr int kGmLdb = kGmCols + 8;

// ---- dx = gather(ddisp) + dlogits @ Wg ------------------------------------------------------
// Block: 8 warps, 64 tokens x 128 columns.  Warp w: tokens 16 (w & 3) .., columns 64 (w >> 2) ..
__global__ void __launch_bounds__(256, 2)
dispatch_bwd_mma_kernel(const __nv_bfloat16* __restrict__ ddisp, const int32_t* __restrict__ idx,
                        const int32_t* __restrict__ slot, const float* __restrict__ dlogits,
                        const __nv_bfloat16* __restrict__ wg, int64_t Ttok, int M, int E, int EP,
                        int k, int C, int Cs, __nv_bfloat16* __restrict__ dx) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lda = EP + 8;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [64][lda]
  __nv_bfloat16* a_lo = a_hi + kGmTok * lda;                              // [64][lda]
  __nv_bfloat16* bs = a_lo + kGmTok * lda;                                // [EP][136]
  float* cs = reinterpret_cast<float*>(smem_raw);                         // [64][132], after the MMAs
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t tok0 = (int64_t)blockIdx.y * kGmTok;
  const int col0 = blockIdx.x * kGmCols;

  // The gathered gradient rows are the kernel's HBM traffic: for k <= 2 their loads are issued
  // first, so that they are in flight while the gate product is staged and computed.
  constexpr int kIt = kGmTok * (kGmCols / 8) / 256;
  const bool early = k <= 2 && ddisp != nullptr;
  uint4 pre[kIt][2];
  uint32_t okmask = 0;               // which of them are rows to add (applied where they are used)
  if (early) {
    // Branch-free, in two rounds: first every (expert, slot) pair this thread needs, then every
    // row vector (rows that were dropped or lie past the end read a valid dummy address and are
    // left out of the sum).  With a branch per row the loads went out one memory round trip after
    // the other, twenty-four per block.
    int sl[kIt][2], ex[kIt][2];
#pragma unroll
    for (int it = 0; it < kIt; ++it) {
      const int64_t t = min(tok0 + ((tid + 256 * it) >> 4), Ttok - 1);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int64_t pi = t * k + min(j, k - 1);
        sl[it][j] = slot[pi];
        ex[it][j] = idx[pi];
      }
    }
    bool ok[kIt][2];
#pragma unroll
    for (int it = 0; it < kIt; ++it) {
      const int w = tid + 256 * it;
      const int c8 = (w & 15) * 8;
      const int64_t t = tok0 + (w >> 4);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        ok[it][j] = t < Ttok && j < k && sl[it][j] < C;
        const int64_t r = ok[it][j] ? (int64_t)ex[it][j] * Cs + sl[it][j] : 0;
        pre[it][j] = *reinterpret_cast<const uint4*>(ddisp + r * M + col0 + c8);
      }
    }
#pragma unroll
    for (int it = 0; it < kIt; ++it)
#pragma unroll
      for (int j = 0; j < 2; ++j) okmask |= (ok[it][j] ? 1u : 0u) << (2 * it + j);
  }

  if (E == EP && EP <= 64 && (E & 3) == 0) {
    // Common case (up to 64 experts): every load of the two operand tiles is issued before the
    // first one is used -- a loop that loads, converts and stores one vector at a time pays a
    // memory round trip per iteration, eight per block.
    const int q4 = EP >> 2;
    float4 dv[4];
    uint4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int tl = i / q4, e = (i - tl * q4) * 4;
      const int64_t t = tok0 + tl;
      dv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < kGmTok * q4 && t < Ttok) dv[u] = *reinterpret_cast<const float4*>(dlogits + t * E + e);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int e = i >> 4, v = i & 15;
      wv[u] = make_uint4(0, 0, 0, 0);
      if (e < E) wv[u] = *reinterpret_cast<const uint4*>(wg + (int64_t)e * M + col0 + v * 8);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int tl = i / q4, e = (i - tl * q4) * 4;
      if (i < kGmTok * q4) {
        __align__(8) __nv_bfloat16 h[4];
        __align__(8) __nv_bfloat16 l[4];
        split_bf16(dv[u].x, h[0], l[0]);
        split_bf16(dv[u].y, h[1], l[1]);
        split_bf16(dv[u].z, h[2], l[2]);
        split_bf16(dv[u].w, h[3], l[3]);
        *reinterpret_cast<uint2*>(a_hi + tl * lda + e) = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(a_lo + tl * lda + e) = *reinterpret_cast<const uint2*>(l);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int e = i >> 4, v = i & 15;
      if (e < EP) *reinterpret_cast<uint4*>(bs + e * kGmLdb + v * 8) = wv[u];
    }
  } else {
    if (E == EP && (E & 3) == 0) {            // four experts per thread and step: 16-byte loads
      const int q4 = EP >> 2;
      for (int i = tid; i < kGmTok * q4; i += 256) {
        const int tl = i / q4, e = (i - tl * q4) * 4;
        const int64_t t = tok0 + tl;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < Ttok) v = *reinterpret_cast<const float4*>(dlogits + t * E + e);
        __align__(8) __nv_bfloat16 h[4];
        __align__(8) __nv_bfloat16 l[4];
        split_bf16(v.x, h[0], l[0]);
        split_bf16(v.y, h[1], l[1]);
        split_bf16(v.z, h[2], l[2]);
        split_bf16(v.w, h[3], l[3]);
        *reinterpret_cast<uint2*>(a_hi + tl * lda + e) = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(a_lo + tl * lda + e) = *reinterpret_cast<const uint2*>(l);
      }
    } else {
      for (int i = tid; i < kGmTok * EP; i += 256) {
        const int tl = i / EP, e = i - tl * EP;
        const int64_t t = tok0 + tl;
        const float v = (t < Ttok && e < E) ? dlogits[t * E + e] : 0.f;
        split_bf16(v, a_hi[tl * lda + e], a_lo[tl * lda + e]);
      }
    }
    for (int i = tid; i < EP * (kGmCols / 8); i += 256) {
      const int e = i >> 4, v = i & 15;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (e < E) w = *reinterpret_cast<const uint4*>(wg + (int64_t)e * M + col0 + v * 8);
      *reinterpret_cast<uint4*>(bs + e * kGmLdb + v * 8) = w;
    }
  }
  __syncthreads();

  const int mt = warp & 3, nh = warp >> 2;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int ks = 0; ks < EP / 16; ++ks) {
    uint32_t ah[4], al[4];
    const int arow = mt * 16 + (lane & 15), acol = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(a_hi + arow * lda + acol, ah);
    ldsm_x4(a_lo + arow * lda + acol, al);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      // four 8x8 blocks of the [k][n] tile: (k 0-7, n 0-7) (k 8-15, n 0-7) (k 0-7, n 8-15) ...
      const int krow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int ncol = nh * 64 + p * 16 + (lane >> 4) * 8;
      uint32_t b[4];
      ldsm_x4_trans(bs + krow * kGmLdb + ncol, b);
      mma16816(acc[2 * p], ah, b[0], b[1]);
      mma16816(acc[2 * p], al, b[0], b[1]);
      mma16816(acc[2 * p + 1], ah, b[2], b[3]);
      mma16816(acc[2 * p + 1], al, b[2], b[3]);
    }
  }
  __syncthreads();                                  // operand tiles are dead: reuse as the C tile
  constexpr int ldc = kGmCols + 4;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      cs[(mt * 16 + g + (j >> 1) * 8) * ldc + nh * 64 + i * 8 + 2 * q + (j & 1)] = acc[i][j];
  __syncthreads();

  // gather pass: a thread owns 8 consecutive columns of one token
#pragma unroll
  for (int it = 0; it < kGmTok * (kGmCols / 8) / 256; ++it) {
    const int w = tid + 256 * it;
    const int tl = w >> 4, c8 = (w & 15) * 8;
    const int64_t t = tok0 + tl;
    if (t >= Ttok) continue;
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = cs[tl * ldc + c8 + c];
    if (early) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t keep = ((okmask >> (2 * it + j)) & 1u) ? 0xffffffffu : 0u;
        const uint32_t wd[4] = {pre[it][j].x & keep, pre[it][j].y & keep, pre[it][j].z & keep,
                                pre[it][j].w & keep};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          v[2 * c] += __uint_as_float(wd[c] << 16);
          v[2 * c + 1] += __uint_as_float(wd[c] & 0xffff0000u);
        }
      }
      Vec16<__nv_bfloat16>::store(dx + t * M + col0 + c8, v);
      continue;
    }
    for (int j = 0; j < k && ddisp != nullptr; ++j) {
      const int s = slot[t * k + j];
      if (s >= C) continue;
      const int64_t r = (int64_t)idx[t * k + j] * Cs + s;
      float d[8];
      Vec16<__nv_bfloat16>::load(ddisp + r * M + col0 + c8, d);
#pragma unroll
      for (int c = 0; c < 8; ++c) v[c] += d[c];
    }
    Vec16<__nv_bfloat16>::store(dx + t * M + col0 + c8, v);
  }
}

// The same product for the common case (top-1 / top-2, up to 64 experts, a gradient to gather):
// every global read of the block is asynchronous.  The (expert, slot) pairs are read first; the Wg
// tile and the gathered rows then travel to shared memory with cp.async (dropped pairs and tokens
// past the end are zero-filled), dlogits through registers (it is split into bf16 hi + lo on the
// way); the MMAs run as soon as the two small operand tiles are there, the gathered rows are only
// waited for in front of the final sum.  No registers hold rows in flight, so three blocks fit an
// SM (69 KB of shared memory each) and one block's stores overlap the next block's loads.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
               ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}
constexpr int kGmGatherBytes = 2 * kGmTok * kGmCols * 2;      // two rows per token, 128 columns

__global__ void __launch_bounds__(256, 3)
dispatch_bwd_mma_async_kernel(const __nv_bfloat16* __restrict__ ddisp, const int32_t* __restrict__ idx,
                              const int32_t* __restrict__ slot, const float* __restrict__ dlogits,
                              const __nv_bfloat16* __restrict__ wg, int64_t Ttok, int M, int E,
                              int k, int C, int Cs, __nv_bfloat16* __restrict__ dx) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int EP = E;
  const int lda = EP + 8;
  __nv_bfloat16* gt = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [2][64][128] gathered rows
  unsigned char* ops = smem_raw + kGmGatherBytes;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(ops);            // [64][lda]
  __nv_bfloat16* a_lo = a_hi + kGmTok * lda;                              // [64][lda]
  __nv_bfloat16* bs = a_lo + kGmTok * lda;                                // [EP][136]
  float* cs = reinterpret_cast<float*>(ops);                              // [64][132], after the MMAs
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t tok0 = (int64_t)blockIdx.y * kGmTok;
  const int col0 = blockIdx.x * kGmCols;
  constexpr int kIt = kGmTok * (kGmCols / 8) / 256;                       // 4

  int sl[kIt][2], ex[kIt][2];
#pragma unroll
  for (int it = 0; it < kIt; ++it) {
    const int64_t t = min(tok0 + ((tid + 256 * it) >> 4), Ttok - 1);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t pi = t * k + min(j, k - 1);
      sl[it][j] = slot[pi];
      ex[it][j] = idx[pi];
    }
  }
  // group 0: the Wg tile
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = tid + 256 * u;
    const int e = i >> 4, v = i & 15;
    if (e < EP) cp_async_16(bs + e * kGmLdb + v * 8, wg + (int64_t)e * M + col0 + v * 8, 16);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  const int q4 = EP >> 2;
  float4 dv[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = tid + 256 * u;
    const int tl = i / q4, e = (i - tl * q4) * 4;
    const int64_t t = tok0 + tl;
    dv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < kGmTok * q4 && t < Ttok) dv[u] = *reinterpret_cast<const float4*>(dlogits + t * E + e);
  }
  // group 1: the gathered rows
#pragma unroll
  for (int it = 0; it < kIt; ++it) {
    const int w = tid + 256 * it;
    const int tl = w >> 4, c8 = (w & 15) * 8;
    const int64_t t = tok0 + tl;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const bool ok = t < Ttok && j < k && sl[it][j] < C;
      const int64_t r = ok ? (int64_t)ex[it][j] * Cs + sl[it][j] : 0;
      cp_async_16(gt + (j * kGmTok + tl) * kGmCols + c8, ddisp + r * M + col0 + c8, ok ? 16 : 0);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = tid + 256 * u;
    const int tl = i / q4, e = (i - tl * q4) * 4;
    if (i < kGmTok * q4) {
      __align__(8) __nv_bfloat16 h[4];
      __align__(8) __nv_bfloat16 l[4];
      split_bf16(dv[u].x, h[0], l[0]);
      split_bf16(dv[u].y, h[1], l[1]);
      split_bf16(dv[u].z, h[2], l[2]);
      split_bf16(dv[u].w, h[3], l[3]);
      *reinterpret_cast<uint2*>(a_hi + tl * lda + e) = *reinterpret_cast<const uint2*>(h);
      *reinterpret_cast<uint2*>(a_lo + tl * lda + e) = *reinterpret_cast<const uint2*>(l);
    }
  }
  asm volatile("cp.async.wait_group 1;" ::: "memory");      // the Wg tile has landed
  __syncthreads();

  const int mt = warp & 3, nh = warp >> 2;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int ks = 0; ks < EP / 16; ++ks) {
    uint32_t ah[4], al[4];
    const int arow = mt * 16 + (lane & 15), acol = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(a_hi + arow * lda + acol, ah);
    ldsm_x4(a_lo + arow * lda + acol, al);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int krow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int ncol = nh * 64 + p * 16 + (lane >> 4) * 8;
      uint32_t b[4];
      ldsm_x4_trans(bs + krow * kGmLdb + ncol, b);
      mma16816(acc[2 * p], ah, b[0], b[1]);
      mma16816(acc[2 * p], al, b[0], b[1]);
      mma16816(acc[2 * p + 1], ah, b[2], b[3]);
      mma16816(acc[2 * p + 1], al, b[2], b[3]);
    }
  }
  __syncthreads();                                  // operand tiles are dead: reuse as the C tile
  constexpr int ldc = kGmCols + 4;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      cs[(mt * 16 + g + (j >> 1) * 8) * ldc + nh * 64 + i * 8 + 2 * q + (j & 1)] = acc[i][j];
  asm volatile("cp.async.wait_group 0;" ::: "memory");      // this thread's gathered vectors
  __syncthreads();

  // final sum: a thread owns 8 consecutive columns of one token (the vectors it fetched itself)
#pragma unroll
  for (int it = 0; it < kIt; ++it) {
    const int w = tid + 256 * it;
    const int tl = w >> 4, c8 = (w & 15) * 8;
    const int64_t t = tok0 + tl;
    if (t >= Ttok) continue;
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = cs[tl * ldc + c8 + c];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 pv = *reinterpret_cast<const uint4*>(gt + (j * kGmTok + tl) * kGmCols + c8);
      const uint32_t wd[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        v[2 * c] += __uint_as_float(wd[c] << 16);
        v[2 * c + 1] += __uint_as_float(wd[c] & 0xffff0000u);
      }
    }
    Vec16<__nv_bfloat16>::store(dx + t * M + col0 + c8, v);
  }
}

int launch_dispatch_bwd_mma(const void* ddisp, const int32_t* idx, const int32_t* slot,
                            const float* dlogits, const void* wg, int64_t T, int M, int E, int k,
                            int C, int Cs, void* dx, cudaStream_t st) {
  const int EP = (E + 15) / 16 * 16;
  const size_t ops = (size_t)(2 * kGmTok * (EP + 8) + EP * kGmLdb) * 2;
  const size_t ctile = (size_t)kGmTok * (kGmCols + 4) * 4;
  const size_t smem = ops > ctile ? ops : ctile;
  static PerDeviceInt configured;      // per device; the attribute only ever needs to grow
  const int dev_ = current_device();
  if ((int64_t)smem > configured.get(dev_)) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(dispatch_bwd_mma_kernel,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set(dev_, (int64_t)smem);
  }
  dim3 grid(M / kGmCols, (unsigned)((T + kGmTok - 1) / kGmTok));
  if (ddisp != nullptr && k <= 2 && E == EP && EP <= 64 && (E & 3) == 0 &&
      (reinterpret_cast<uintptr_t>(ddisp) & 15) == 0 && (reinterpret_cast<uintptr_t>(wg) & 15) == 0) {
    const size_t asmem = kGmGatherBytes + smem;
    static PerDeviceInt aconfigured;
    if ((int64_t)asmem > aconfigured.get(dev_)) {
      MOLE_CUDA_OK(cudaFuncSetAttribute(dispatch_bwd_mma_async_kernel,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)asmem));
      aconfigured.set(dev_, (int64_t)asmem);
    }
    dispatch_bwd_mma_async_kernel<<<grid, 256, asmem, st>>>(
        static_cast<const __nv_bfloat16*>(ddisp), idx, slot, dlogits,
        static_cast<const __nv_bfloat16*>(wg), T, M, E, k, C, Cs, static_cast<__nv_bfloat16*>(dx));
    MOLE_LAUNCH_OK();
    return MOLE_OK;
  }
  dispatch_bwd_mma_kernel<<<grid, 256, smem, st>>>(
      static_cast<const __nv_bfloat16*>(ddisp), idx, slot, dlogits,
      static_cast<const __nv_bfloat16*>(wg), T, M, E, EP, k, C, Cs, static_cast<__nv_bfloat16*>(dx));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// ---- partial[chunk] = dlogits[chunk]^T @ x[chunk] ---------------------------------------------
// Block: 8 warps, all experts x 128 columns, `chunk` tokens in sub-chunks of 64; the block's
// partial product goes to partial[blockIdx.y] (the caller adds the chunks in a fixed order, so the
// gradient is bit-reproducible).  The chunk is sized for about two blocks per SM.  Warp w: columns 64 (w >> 2) ..,
// expert tiles (w & 3) + 4 i.  Both operands sit in shared memory token-major ([k][m], [k][n]),
// so both fragments come from transposing ldmatrix loads.
template <int MT>                       // expert tiles of 16 per warp: EP <= 64 * MT
__global__ void __launch_bounds__(256)
gate_wgrad_mma_kernel(const float* __restrict__ dlogits, const __nv_bfloat16* __restrict__ x,
                      int64_t Ttok, int M, int E, int EP, int chunk, float* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lda = EP + 8;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [64 tok][lda]
  __nv_bfloat16* a_lo = a_hi + kGmTok * lda;
  __nv_bfloat16* xs = a_lo + kGmTok * lda;                                // [64 tok][136]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mg = warp & 3, nh = warp >> 2;
  const int col0 = blockIdx.x * kGmCols;
  const int64_t chunk0 = (int64_t)blockIdx.y * chunk;
  float acc[MT][8][4];
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][i][j] = 0.f;

  // Up to 64 experts (MT == 1, the common case): the loads of a sub-chunk's two operand tiles are
  // all issued at once, one sub-chunk ahead, and wait in registers while the previous sub-chunk is
  // multiplied -- a loop that loads, converts and stores one vector at a time pays a memory round
  // trip per iteration (eight per sub-chunk, 6 us where the data needs 1 us).
  const bool fast = MT == 1 && E == EP && (E & 3) == 0;
  const int q4 = EP >> 2;
  float4 dv[4];
  uint4 xv[4];
  auto fetch = [&](int64_t tok0) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int tl = i / q4, e = (i - tl * q4) * 4;
      const int64_t t = tok0 + tl;
      dv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < kGmTok * q4 && t < Ttok) dv[u] = *reinterpret_cast<const float4*>(dlogits + t * E + e);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + 256 * u;
      const int tl = i >> 4, v = i & 15;
      const int64_t t = tok0 + tl;
      xv[u] = make_uint4(0, 0, 0, 0);
      if (t < Ttok) xv[u] = *reinterpret_cast<const uint4*>(x + t * M + col0 + v * 8);
    }
  };
  if (fast && chunk0 < Ttok) fetch(chunk0);

  for (int sub = 0; sub < chunk / kGmTok; ++sub) {
    const int64_t tok0 = chunk0 + sub * kGmTok;
    if (tok0 >= Ttok) break;                                  // block-uniform
    if (fast) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = tid + 256 * u;
        const int tl = i / q4, e = (i - tl * q4) * 4;
        if (i < kGmTok * q4) {
          __align__(8) __nv_bfloat16 h[4];
          __align__(8) __nv_bfloat16 l[4];
          split_bf16(dv[u].x, h[0], l[0]);
          split_bf16(dv[u].y, h[1], l[1]);
          split_bf16(dv[u].z, h[2], l[2]);
          split_bf16(dv[u].w, h[3], l[3]);
          *reinterpret_cast<uint2*>(a_hi + tl * lda + e) = *reinterpret_cast<const uint2*>(h);
          *reinterpret_cast<uint2*>(a_lo + tl * lda + e) = *reinterpret_cast<const uint2*>(l);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = tid + 256 * u;
        *reinterpret_cast<uint4*>(xs + (i >> 4) * kGmLdb + (i & 15) * 8) = xv[u];
      }
      __syncthreads();
      if (sub + 1 < chunk / kGmTok && tok0 + kGmTok < Ttok) fetch(tok0 + kGmTok);
    } else {
    if (E == EP && (E & 3) == 0) {          // four experts per thread and step: 16-byte loads
      for (int i = tid; i < kGmTok * q4; i += 256) {
        const int tl = i / q4, e = (i - tl * q4) * 4;
        const int64_t t = tok0 + tl;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < Ttok) v = *reinterpret_cast<const float4*>(dlogits + t * E + e);
        __align__(8) __nv_bfloat16 h[4];
        __align__(8) __nv_bfloat16 l[4];
        split_bf16(v.x, h[0], l[0]);
        split_bf16(v.y, h[1], l[1]);
        split_bf16(v.z, h[2], l[2]);
        split_bf16(v.w, h[3], l[3]);
        *reinterpret_cast<uint2*>(a_hi + tl * lda + e) = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(a_lo + tl * lda + e) = *reinterpret_cast<const uint2*>(l);
      }
    } else {
      for (int i = tid; i < kGmTok * EP; i += 256) {
        const int tl = i / EP, e = i - tl * EP;
        const int64_t t = tok0 + tl;
        const float v = (t < Ttok && e < E) ? dlogits[t * E + e] : 0.f;
        split_bf16(v, a_hi[tl * lda + e], a_lo[tl * lda + e]);
      }
    }
    for (int i = tid; i < kGmTok * (kGmCols / 8); i += 256) {
      const int tl = i >> 4, v = i & 15;
      const int64_t t = tok0 + tl;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (t < Ttok) w = *reinterpret_cast<const uint4*>(x + t * M + col0 + v * 8);
      *reinterpret_cast<uint4*>(xs + tl * kGmLdb + v * 8) = w;
    }
    __syncthreads();
    }
#pragma unroll
    for (int ks = 0; ks < kGmTok / 16; ++ks) {
      uint32_t b[4][4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int krow = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int ncol = nh * 64 + p * 16 + (lane >> 4) * 8;
        ldsm_x4_trans(xs + krow * kGmLdb + ncol, b[p]);
      }
#pragma unroll
      for (int a = 0; a < MT; ++a) {
        const int m0 = (mg + 4 * a) * 16;
        if (m0 >= EP) continue;                               // warp-uniform
        // A[m][k] from [k][m] storage: blocks (m 0-7, k 0-7) (m 8-15, k 0-7) (m 0-7, k 8-15) ...
        const int krow = ks * 16 + (lane >> 4) * 8 + (lane & 7);
        const int mcol = m0 + ((lane >> 3) & 1) * 8;
        uint32_t ah[4], al[4];
        ldsm_x4_trans(a_hi + krow * lda + mcol, ah);
        ldsm_x4_trans(a_lo + krow * lda + mcol, al);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          mma16816(acc[a][2 * p], ah, b[p][0], b[p][1]);
          mma16816(acc[a][2 * p], al, b[p][0], b[p][1]);
          mma16816(acc[a][2 * p + 1], ah, b[p][2], b[p][3]);
          mma16816(acc[a][2 * p + 1], al, b[p][2], b[p][3]);
        }
      }
    }
    __syncthreads();
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = (mg + 4 * a) * 16 + g + (j >> 1) * 8;
        const int m = col0 + nh * 64 + i * 8 + 2 * q + (j & 1);
        if (e < E) partial[((int64_t)blockIdx.y * E + e) * M + m] = acc[a][i][j];
      }
}

template <int MT>
static int launch_wgrad_mma_t(const float* dlogits, const void* x, int64_t T, int M, int E, int EP,
                              int chunk, int n_chunks, float* partial, cudaStream_t st) {
  const size_t smem = (size_t)(2 * kGmTok * (EP + 8) + kGmTok * kGmLdb) * 2;
  auto kern = gate_wgrad_mma_kernel<MT>;
  static PerDeviceInt configured;      // per device; the attribute only ever needs to grow
  const int dev_ = current_device();
  if ((int64_t)smem > configured.get(dev_)) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set(dev_, (int64_t)smem);
  }
  dim3 grid(M / kGmCols, (unsigned)n_chunks);
  kern<<<grid, 256, smem, st>>>(dlogits, static_cast<const __nv_bfloat16*>(x), T, M, E, EP, chunk,
                                partial);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

int launch_gate_wgrad_mma(const float* dlogits, const void* x, int64_t T, int M, int E, int chunk,
                          int n_chunks, float* partial, cudaStream_t st) {
  const int EP = (E + 15) / 16 * 16;
  if (EP <= 64) return launch_wgrad_mma_t<1>(dlogits, x, T, M, E, EP, chunk, n_chunks, partial, st);
  if (EP <= 128) return launch_wgrad_mma_t<2>(dlogits, x, T, M, E, EP, chunk, n_chunks, partial, st);
  return launch_wgrad_mma_t<4>(dlogits, x, T, M, E, EP, chunk, n_chunks, partial, st);
}

}  // namespace mole
