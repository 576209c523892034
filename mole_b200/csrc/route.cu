// (a) Gate and routing-index build.
//
// gate_topk_kernel     x @ Wg^T (+bias) -> softmax -> top-k, per-block expert histograms and
//                      per-block partial score sums.  Replaces MOLETopk.forward
//                      (MOLE/utils/Ugate.py:11-14) and the selection half of the
//                      extract_critical call (MOLE/moe/layer.py:445-447).
// route_scan_kernel    ordered exclusive scan of the histograms over (choice, token block):
//                      slot bases, counts = min(hist, C), offsets, first-choice histogram, l_aux.
// route_slot_kernel    slot of every (token, choice) pair, kept mask folded into the gate
//                      weights, token permutation.
// gate_bwd_kernel      dlogits from d(gates) and d(l_aux).
// gate_wgrad_kernel    dWg += dlogits^T @ x (split over tokens, fp32 atomics).
//
// All integer outputs are produced by integer arithmetic in a fixed order: no atomics decide
// a slot, so the result is a pure function of the scores.
#include <mutex>

#include "common.cuh"

namespace mole {

constexpr int kGateTok = 64;     // tokens per block in every routing kernel
constexpr int kGateKC = 32;      // K chunk of the gate GEMM
constexpr int kGateThreads = 256;
constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Second half of the gate kernel, also used on caller-provided scores.
// ls: [kGateTok][E + 1] fp32 in shared memory holding logits (softmax_needed) or scores.
// kPerLane = experts a lane holds (ceil(E / 32), rounded up to 1, 2, 4 or 8): the loops over a
// lane's experts are unrolled to exactly that, not to the largest expert count the library takes.
template <int kPerLane>
__device__ void softmax_topk_lanes(float* ls, int* hist_s, int64_t tok0, int64_t T, int E, int k,
                                   int normalize, bool softmax_needed, float* scores,
                                   int32_t* idx, float* gates, int32_t* hist, float* me_part,
                                   int nblk) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ldl = E + 1;
  for (int i = tid; i < k * E; i += kGateThreads) hist_s[i] = 0;
  __syncthreads();

  static_assert(kPerLane * 32 <= kMaxExperts, "more experts per lane than the library takes");
  for (int tt = 0; tt < kGateTok / 8; ++tt) {
    const int tl = warp * (kGateTok / 8) + tt;
    const int64_t t = tok0 + tl;
    if (t >= T) break;           // warp-uniform
    float v[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? ls[tl * ldl + e] : -INFINITY;
    }
    if (softmax_needed) {
      float m = v[0];
#pragma unroll
      for (int j = 1; j < kPerLane; ++j) m = fmaxf(m, v[j]);
      m = warp_max(m);
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        v[j] = (lane + 32 * j) < E ? expf(v[j] - m) : 0.f;
        s += v[j];
      }
      s = warp_sum(s);
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        const int e = lane + 32 * j;
        v[j] = v[j] / s;
        if (e < E) {
          ls[tl * ldl + e] = v[j];
          scores[t * E + e] = v[j];
        } else {
          v[j] = -INFINITY;
        }
      }
    }
    // top-k on the scores: largest value, ties to the lower expert id
    float gsel[kMaxTopK];
    int esel[kMaxTopK];
    float gsum = 0.f;
    for (int c = 0; c < k; ++c) {
      float bv = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {      // ascending e: strict > keeps the lower id
        if (v[j] > bv) { bv = v[j]; be = lane + 32 * j; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
#pragma unroll
      for (int j = 0; j < kPerLane; ++j)
        if (lane + 32 * j == be) v[j] = -INFINITY;
      gsel[c] = bv;
      esel[c] = be;
      gsum += bv;
    }
    if (lane == 0) {
      const float inv = normalize ? 1.0f / fmaxf(gsum, 1e-9f) : 1.0f;
      for (int c = 0; c < k; ++c) {
        idx[t * k + c] = esel[c];
        gates[t * k + c] = normalize ? gsel[c] * inv : gsel[c];
        atomicAdd(&hist_s[c * E + esel[c]], 1);
      }
    }
  }
  __syncthreads();
  const int blk = blockIdx.x;
  // expert-major layouts: the scan kernel reads one expert's (choice, block) sequence contiguously
  for (int i = tid; i < k * E; i += kGateThreads) {
    const int c = i / E, e = i - c * E;
    hist[((int64_t)e * k + c) * nblk + blk] = hist_s[i];
  }
  const int nvalid = (int)min((int64_t)kGateTok, T - tok0);
  for (int e = tid; e < E; e += kGateThreads) {
    float s = 0.f;
    for (int tl = 0; tl < nvalid; ++tl) s += ls[tl * ldl + e];
    me_part[(int64_t)e * nblk + blk] = s;
  }
}

__device__ __forceinline__ void softmax_topk_block(float* ls, int* hist_s, int64_t tok0, int64_t T,
                                                   int E, int k, int normalize, bool softmax_needed,
                                                   float* scores, int32_t* idx, float* gates,
                                                   int32_t* hist, float* me_part, int nblk) {
  if (E <= 32)
    softmax_topk_lanes<1>(ls, hist_s, tok0, T, E, k, normalize, softmax_needed, scores, idx, gates, hist, me_part, nblk);
  else if (E <= 64)
    softmax_topk_lanes<2>(ls, hist_s, tok0, T, E, k, normalize, softmax_needed, scores, idx, gates, hist, me_part, nblk);
  else if (E <= 128)
    softmax_topk_lanes<4>(ls, hist_s, tok0, T, E, k, normalize, softmax_needed, scores, idx, gates, hist, me_part, nblk);
  else
    softmax_topk_lanes<kMaxExperts / 32>(ls, hist_s, tok0, T, E, k, normalize, softmax_needed, scores, idx, gates, hist, me_part, nblk);
}

template <typename T, int EJ>
__global__ void __launch_bounds__(kGateThreads)
gate_topk_kernel(const T* __restrict__ x, const T* __restrict__ wg, const float* __restrict__ bias,
                 int64_t Ttok, int M, int E, int k, int normalize, float* __restrict__ scores,
                 int32_t* __restrict__ idx, float* __restrict__ gates, int32_t* __restrict__ hist,
                 float* __restrict__ me_part, int nblk) {
  extern __shared__ float smem[];
  constexpr int LD = kGateKC + 1;
  float* xs = smem;                              // [64][33]
  float* ws = smem + kGateTok * LD;              // [EJ*16][33]
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int64_t tok0 = (int64_t)blockIdx.x * kGateTok;

  float acc[4][EJ];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < EJ; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < M; k0 += kGateKC) {
#pragma unroll
    for (int r = 0; r < kGateTok * kGateKC / kGateThreads; ++r) {
      const int i = tid + kGateThreads * r;
      const int tl = i >> 5, kk = i & 31;
      const int64_t t = tok0 + tl;
      float v = 0.f;
      if (t < Ttok && k0 + kk < M) v = Elem<T>::to_f(x[t * M + k0 + kk]);
      xs[tl * LD + kk] = v;
    }
#pragma unroll
    for (int r = 0; r < EJ * 16 * kGateKC / kGateThreads; ++r) {
      const int i = tid + kGateThreads * r;
      const int e = i >> 5, kk = i & 31;
      float v = 0.f;
      if (e < E && k0 + kk < M) v = Elem<T>::to_f(wg[(int64_t)e * M + k0 + kk]);
      ws[e * LD + kk] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kGateKC; ++kk) {
      float a[4], b[EJ];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[(ty * 4 + i) * LD + kk];
#pragma unroll
      for (int j = 0; j < EJ; ++j) b[j] = ws[(tx + 16 * j) * LD + kk];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < EJ; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  // logits tile to shared memory (the operand tiles are dead now)
  float* ls = smem;
  const int ldl = E + 1;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < EJ; ++j) {
      const int e = tx + 16 * j;
      if (e < E) ls[(ty * 4 + i) * ldl + e] = acc[i][j] + (bias ? bias[e] : 0.f);
    }
  int* hist_s = reinterpret_cast<int*>(smem + kGateTok * ldl);
  __syncthreads();
  softmax_topk_block(ls, hist_s, tok0, Ttok, E, k, normalize, true, scores, idx, gates, hist,
                     me_part, nblk);
}

// ---- bf16 gate on the warp-level tensor-core path ------------------------------------------
// The gate product is [T, M] x [M, E] with E <= 256: far too small for a tcgen05 tile pipeline to
// pay off, but on CUDA cores it is FMA-bound at ~3 % of the HBM rate it should run at.  Warp-level
// mma.sync (m16n8k16, bf16 in, fp32 accumulate in the hardware's fixed order) brings it to the
// memory roofline: the kernel streams x once through a four-stage cp.async ring.
// Block: 8 warps, 64 tokens; warp w owns tokens 16 * (w & 3) .. +15 and half of the experts.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
               ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(const void* p, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kMmaKC = 64;            // K elements per stage
constexpr int kMmaLds = kMmaKC + 8;   // padded row (144 bytes): conflict-free ldmatrix
constexpr int kMmaStages = 4;         // cp.async ring: one block per SM has nothing else to hide latency

template <int NT>                     // expert tiles of 8: experts padded to NT * 8 >= 32
__global__ void __launch_bounds__(kGateThreads)
gate_topk_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg,
                     const float* __restrict__ bias, int64_t Ttok, int M, int E, int k,
                     int normalize, float* __restrict__ scores, int32_t* __restrict__ idx,
                     float* __restrict__ gates, int32_t* __restrict__ hist,
                     float* __restrict__ me_part, int nblk) {
  extern __shared__ float smem[];
  constexpr int EP = NT * 8, NTW = NT / 2;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);          // [stages][64][72]
  __nv_bfloat16* wsm = xs + kMmaStages * kGateTok * kMmaLds;           // [stages][EP][72]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mt = warp & 3, nh = warp >> 2;
  const int64_t tok0 = (int64_t)blockIdx.x * kGateTok;

  auto load_chunk = [&](int c, int st) {
    for (int i = tid; i < kGateTok * 8; i += kGateThreads) {
      const int r = i >> 3, v = i & 7;
      const int64_t t = tok0 + r;
      const bool ok = t < Ttok;
      cp_async16(xs + (st * kGateTok + r) * kMmaLds + v * 8,
                 x + (ok ? t : 0) * M + c * kMmaKC + v * 8, ok ? 16 : 0);
    }
    for (int i = tid; i < EP * 8; i += kGateThreads) {
      const int r = i >> 3, v = i & 7;
      const bool ok = r < E;
      cp_async16(wsm + (st * EP + r) * kMmaLds + v * 8,
                 wg + (int64_t)(ok ? r : 0) * M + c * kMmaKC + v * 8, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int nchunks = M / kMmaKC;
  // one commit group per chunk slot (empty past the end), so "all but the newest stages - 2
  // groups are complete" always means chunk c has landed
#pragma unroll
  for (int c = 0; c < kMmaStages - 1; ++c) {
    if (c < nchunks) load_chunk(c, c);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int c = 0; c < nchunks; ++c) {
    const int st = c % kMmaStages;
    asm volatile("cp.async.wait_group %0;" ::"n"(kMmaStages - 2) : "memory");
    __syncthreads();                       // chunk c visible; stage of chunk c - 1 free again
    if (c + kMmaStages - 1 < nchunks) load_chunk(c + kMmaStages - 1, (c + kMmaStages - 1) % kMmaStages);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const __nv_bfloat16* xa = xs + st * kGateTok * kMmaLds;
    const __nv_bfloat16* wb = wsm + st * EP * kMmaLds;
#pragma unroll
    for (int ks = 0; ks < kMmaKC / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(xa + (mt * 16 + (lane & 15)) * kMmaLds + ks * 16 + (lane >> 4) * 8, a);
#pragma unroll
      for (int p = 0; p < NTW / 2; ++p) {
        const int n0 = (nh * NTW + 2 * p) * 8;
        uint32_t b[4];
        ldmatrix_x4(wb + (n0 + (lane & 7) + ((lane >> 4) << 3)) * kMmaLds + ks * 16 +
                        ((lane >> 3) & 1) * 8, b);
        mma_bf16_16816(acc[2 * p], a, b[0], b[1]);
        mma_bf16_16816(acc[2 * p + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  // logits tile to shared memory (operand stages are dead after the last barrier)
  float* ls = smem;
  const int ldl = E + 1;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < NTW; ++i) {
    const int e0 = (nh * NTW + i) * 8 + 2 * q;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + (j & 1), row = mt * 16 + g + (j >> 1) * 8;
      if (e < E) ls[row * ldl + e] = acc[i][j] + (bias ? bias[e] : 0.f);
    }
  }
  int* hist_s = reinterpret_cast<int*>(smem + kGateTok * ldl);
  __syncthreads();
  softmax_topk_block(ls, hist_s, tok0, Ttok, E, k, normalize, true, scores, idx, gates, hist,
                     me_part, nblk);
}

__global__ void __launch_bounds__(kGateThreads)
topk_from_scores_kernel(const float* __restrict__ scores, int64_t Ttok, int E, int k,
                        int normalize, int32_t* __restrict__ idx, float* __restrict__ gates,
                        int32_t* __restrict__ hist, float* __restrict__ me_part, int nblk) {
  extern __shared__ float smem[];
  float* ls = smem;
  const int ldl = E + 1;
  const int64_t tok0 = (int64_t)blockIdx.x * kGateTok;
  for (int i = threadIdx.x; i < kGateTok * E; i += kGateThreads) {
    const int tl = i / E, e = i - tl * E;
    const int64_t t = tok0 + tl;
    ls[tl * ldl + e] = t < Ttok ? scores[t * E + e] : 0.f;
  }
  int* hist_s = reinterpret_cast<int*>(smem + kGateTok * ldl);
  __syncthreads();
  softmax_topk_block(ls, hist_s, tok0, Ttok, E, k, normalize, false, nullptr, idx, gates, hist,
                     me_part, nblk);
}

// One block of 32 warps.  hist [E][k][nblk] is turned in place into the slot base of every
// (expert, choice, block): all earlier choices of all tokens, then earlier blocks.  A warp owns
// an expert at a time and scans its k * nblk sequence 32 values per step.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
route_scan_kernel(int32_t* __restrict__ hist, const float* __restrict__ me_part, int64_t T,
                  int E, int k, int C, int nblk, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ first_hist,
                  float* __restrict__ l_aux, int32_t* __restrict__ perm) {
  __shared__ float prod[kMaxExperts];
  __shared__ int cnt[kMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = k * nblk;
  // perm starts as "no pair" everywhere (the slot kernel behind this one fills the kept pairs):
  // done here instead of by a memset launch of its own
  for (int64_t i = threadIdx.x; i < T * k; i += kScanThreads) perm[i] = -1;
  for (int e = warp; e < E; e += kScanThreads / 32) {
    int32_t* h = hist + (int64_t)e * n;
    int running = 0, first = 0;
    // eight steps of 32 values are loaded at once: one memory round trip per 256 values
    for (int i00 = 0; i00 < n; i00 += 256) {
      int vv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i00 + 32 * j + lane;
        vv[j] = i < n ? h[i] : 0;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i0 = i00 + 32 * j;
        if (i0 >= n) break;                       // warp-uniform
        const int i = i0 + lane;
        const int v = vv[j];
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += u;
        }
        const int excl = running + incl - v;
        if (i < n) h[i] = excl;
        if (i == nblk) first = excl;              // everything of choice 0
        running += __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    first = __reduce_max_sync(0xffffffffu, first);
    if (k == 1) first = running;
    // mean score of the expert: lane-strided partial sums, then a fixed shuffle tree
    float me = 0.f;
    for (int b = lane; b < nblk; b += 32) me += me_part[(int64_t)e * nblk + b];
    me = warp_sum(me);
    if (lane == 0) {
      const float fT = (float)T;
      prod[e] = (me / fT) * ((float)first / fT);
      cnt[e] = min(running, C);
      counts[e] = cnt[e];
      first_hist[e] = first;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    float s = 0.f;
    for (int i = 0; i < E; ++i) {
      offsets[i] = off;
      off += cnt[i];
      s += prod[i];
    }
    offsets[E] = off;
    *l_aux = (float)E * s;
  }
}

__global__ void __launch_bounds__(kGateTok)
route_slot_kernel(const int32_t* __restrict__ idx, const int32_t* __restrict__ base,
                  const int32_t* __restrict__ offsets, int64_t T, int E, int k, int C, int nblk,
                  int32_t* __restrict__ slot, float* __restrict__ gates,
                  int32_t* __restrict__ perm) {
  __shared__ int cnt0[kMaxExperts];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = (int64_t)blockIdx.x * kGateTok + tid;
  for (int c = 0; c < k; ++c) {
    for (int i = tid; i < E; i += kGateTok) cnt0[i] = 0;
    __syncthreads();
    const int e = t < T ? idx[t * k + c] : -1 - lane;       // inactive lanes never match
    const unsigned mask = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(mask & ((1u << lane) - 1u));
    if (warp == 0 && rank == 0 && e >= 0) cnt0[e] = __popc(mask);
    __syncthreads();
    if (t < T) {
      const int s = base[((int64_t)e * k + c) * nblk + blockIdx.x] + (warp == 1 ? cnt0[e] : 0) + rank;
      slot[t * k + c] = s;
      if (s < C) {
        perm[offsets[e] + s] = (int32_t)(t * k + c);
      } else {
        gates[t * k + c] = 0.f;
      }
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
gate_bwd_kernel(const float* __restrict__ scores, const int32_t* __restrict__ idx,
                const int32_t* __restrict__ slot, const float* __restrict__ dgates,
                const float* __restrict__ d_l_aux, const int32_t* __restrict__ first_hist,
                int64_t T, int E, int k, int C, int normalize, float* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  constexpr int kPerLane = kMaxExperts / 32;
  const float fT = (float)T;
  const float coef = d_l_aux ? (*d_l_aux) * (float)E / (fT * fT) : 0.f;
  float s[kPerLane], ds[kPerLane];
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? scores[t * E + e] : 0.f;
    ds[j] = e < E ? coef * (float)first_hist[e] : 0.f;
  }
  float S = 1.f, a = 0.f;
  if (normalize) {
    S = 0.f;
    for (int c = 0; c < k; ++c) S += scores[t * E + idx[t * k + c]];
    S = fmaxf(S, 1e-9f);
    for (int c = 0; c < k; ++c) {
      const bool kept = slot[t * k + c] < C;
      if (kept) a += dgates[t * k + c] * scores[t * E + idx[t * k + c]] / S;
    }
  }
  for (int c = 0; c < k; ++c) {
    const int e = idx[t * k + c];
    const bool kept = slot[t * k + c] < C;
    float d = kept ? dgates[t * k + c] : 0.f;
    if (normalize) d = (d - a) / S;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j)
      if (lane + 32 * j == e) ds[j] += d;
  }
  float inner = 0.f;
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) inner += s[j] * ds[j];
  inner = warp_sum(inner);
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = lane + 32 * j;
    if (e < E) dlogits[t * E + e] = s[j] * (ds[j] - inner);
  }
}

// dWg[e, m] += sum_t dlogits[t, e] * x[t, m], in two stages so that the sum has one fixed order
// (bit-reproducible from run to run): block (column block, token chunk) writes its partial
// [E, 64 columns] product into partial[chunk], gate_wgrad_reduce_kernel then adds the chunks to
// dWg in chunk order.  Block: `chunk` tokens x 64 columns, all experts.
constexpr int kWgTok = 128, kWgCols = 64, kWgKC = 32;
template <typename T, int EJ>
__global__ void __launch_bounds__(256)
gate_wgrad_kernel(const float* __restrict__ dlogits, const T* __restrict__ x, int64_t Ttok, int M,
                  int E, int chunk, float* __restrict__ partial) {
  __shared__ float dl_s[kWgKC][EJ * 16 + 1];
  __shared__ float x_s[kWgKC][kWgCols + 1];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;   // ty: expert group, tx: columns
  const int col0 = blockIdx.x * kWgCols;
  const int64_t tok0 = (int64_t)blockIdx.y * chunk;
  float acc[EJ][4];
#pragma unroll
  for (int j = 0; j < EJ; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
  for (int t0 = 0; t0 < chunk && tok0 + t0 < Ttok; t0 += kWgKC) {
    for (int i = tid; i < kWgKC * EJ * 16; i += 256) {
      const int tl = i / (EJ * 16), e = i - tl * (EJ * 16);
      const int64_t t = tok0 + t0 + tl;
      dl_s[tl][e] = (t < Ttok && e < E) ? dlogits[t * E + e] : 0.f;
    }
    for (int i = tid; i < kWgKC * kWgCols; i += 256) {
      const int tl = i / kWgCols, c = i - tl * kWgCols;
      const int64_t t = tok0 + t0 + tl;
      x_s[tl][c] = (t < Ttok && col0 + c < M) ? Elem<T>::to_f(x[t * M + col0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int tl = 0; tl < kWgKC; ++tl) {
      float a[EJ], b[4];
#pragma unroll
      for (int j = 0; j < EJ; ++j) a[j] = dl_s[tl][ty + 16 * j];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = x_s[tl][tx + 16 * c];
#pragma unroll
      for (int j = 0; j < EJ; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = fmaf(a[j], b[c], acc[j][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < EJ; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int e = ty + 16 * j, m = col0 + tx + 16 * c;
      if (e < E && m < M) partial[((int64_t)blockIdx.y * E + e) * M + m] = acc[j][c];
    }
}

__global__ void gate_wgrad_reduce_kernel(const float* __restrict__ partial, int n_chunks, int64_t n,
                                         float* __restrict__ dwg) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = dwg[i];
  for (int c = 0; c < n_chunks; ++c) s += partial[(int64_t)c * n + i];
  dwg[i] = s;
}

// ---- host side ---------------------------------------------------------------------
static inline int nblocks(int64_t T) { return (int)((T + kGateTok - 1) / kGateTok); }

static int check_route_args(int64_t T, int E, int k, int C) {
  MOLE_REQUIRE(T > 0 && T < (int64_t)1 << 30, "T=%lld out of range", (long long)T);
  MOLE_REQUIRE(E >= 1 && E <= kMaxExperts, "E=%d not in [1,%d]", E, kMaxExperts);
  MOLE_REQUIRE(k >= 1 && k <= kMaxTopK && k <= E, "k=%d not in [1,min(E,%d)]", k, kMaxTopK);
  MOLE_REQUIRE(C >= 1, "capacity %d < 1", C);
  MOLE_REQUIRE(T * k < (int64_t)1 << 31, "T*k overflows int32");
  return MOLE_OK;
}

struct RouteWs {
  int32_t* hist;
  float* me_part;
};
static int64_t route_ws_bytes(int64_t T, int E, int k) {
  const int64_t nb = nblocks(T);
  return ((int64_t)k * nb * E + nb * E) * 4;
}
static RouteWs carve(void* ws, int64_t T, int E, int k) {
  const int64_t nb = nblocks(T);
  RouteWs r;
  r.hist = static_cast<int32_t*>(ws);
  r.me_part = reinterpret_cast<float*>(r.hist + (int64_t)k * nb * E);
  return r;
}

static int route_tail(RouteWs w, int64_t T, int E, int k, int C, int32_t* idx, int32_t* slot,
                      float* gates, int32_t* counts, int32_t* offsets, int32_t* perm,
                      int32_t* first_hist, float* l_aux, cudaStream_t st) {
  const int nb = nblocks(T);
  route_scan_kernel<<<1, kScanThreads, 0, st>>>(w.hist, w.me_part, T, E, k, C, nb, counts, offsets,
                                               first_hist, l_aux, perm);
  MOLE_LAUNCH_OK();
  route_slot_kernel<<<nb, kGateTok, 0, st>>>(idx, w.hist, offsets, T, E, k, C, nb, slot, gates,
                                             perm);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

template <typename T, int EJ>
static int launch_gate(const void* x, const void* wg, const float* bias, int64_t Ttok, int M, int E,
                       int k, int normalize, float* scores, int32_t* idx, float* gates, RouteWs w,
                       cudaStream_t st) {
  const int nb = nblocks(Ttok);
  const size_t tiles = (size_t)(kGateTok + EJ * 16) * (kGateKC + 1) * 4;
  const size_t tail = (size_t)kGateTok * (E + 1) * 4 + (size_t)k * E * 4;
  const size_t smem = tiles > tail ? tiles : tail;
  auto kern = gate_topk_kernel<T, EJ>;
  MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<nb, kGateThreads, smem, st>>>(static_cast<const T*>(x), static_cast<const T*>(wg), bias,
                                       Ttok, M, E, k, normalize, scores, idx, gates, w.hist,
                                       w.me_part, nb);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

template <int NT>
static int launch_gate_mma(const void* x, const void* wg, const float* bias, int64_t Ttok, int M,
                           int E, int k, int normalize, float* scores, int32_t* idx, float* gates,
                           RouteWs w, cudaStream_t st) {
  const int nb = nblocks(Ttok);
  const size_t tiles = (size_t)kMmaStages * (kGateTok + NT * 8) * kMmaLds * 2;
  const size_t tail = (size_t)kGateTok * (E + 1) * 4 + (size_t)k * E * 4;
  const size_t smem = tiles > tail ? tiles : tail;
  auto kern = gate_topk_mma_kernel<NT>;
  static PerDeviceInt configured;      // per device; the attribute only ever needs to grow
  const int dev_ = current_device();
  if ((int64_t)smem > configured.get(dev_)) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set(dev_, (int64_t)smem);
  }
  kern<<<nb, kGateThreads, smem, st>>>(static_cast<const __nv_bfloat16*>(x),
                                       static_cast<const __nv_bfloat16*>(wg), bias, Ttok, M, E, k,
                                       normalize, scores, idx, gates, w.hist, w.me_part, nb);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

static int dispatch_gate_mma(int E, const void* x, const void* wg, const float* bias, int64_t Ttok,
                             int M, int k, int normalize, float* scores, int32_t* idx, float* gates,
                             RouteWs w, cudaStream_t st) {
  if (E <= 32) return launch_gate_mma<4>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  if (E <= 64) return launch_gate_mma<8>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  if (E <= 128) return launch_gate_mma<16>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  return launch_gate_mma<32>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
}

template <typename T>
static int dispatch_gate(int E, const void* x, const void* wg, const float* bias, int64_t Ttok,
                         int M, int k, int normalize, float* scores, int32_t* idx, float* gates,
                         RouteWs w, cudaStream_t st) {
  const int ej = (E + 15) / 16;
  if (ej <= 1) return launch_gate<T, 1>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  if (ej <= 2) return launch_gate<T, 2>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  if (ej <= 4) return launch_gate<T, 4>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  if (ej <= 8) return launch_gate<T, 8>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
  return launch_gate<T, 16>(x, wg, bias, Ttok, M, E, k, normalize, scores, idx, gates, w, st);
}

// Gate kernel by element type and alignment, then the routing-index build, over the scratch `w`
// (a caller workspace or the library's built-in array).
static int gate_route_on(RouteWs w, const void* x, const void* wg, const float* logit_bias, int64_t T,
                         int M, int E, int k, int C, int normalize_gate, int dtype, float* scores,
                         int32_t* idx, int32_t* slot, float* gates, int32_t* counts,
                         int32_t* offsets, int32_t* perm, int32_t* first_hist, float* l_aux,
                         cudaStream_t st) {
  int rc;
  if (dtype == MOLE_F32)
    rc = dispatch_gate<float>(E, x, wg, logit_bias, T, M, k, normalize_gate, scores, idx, gates, w, st);
  else if (dtype == MOLE_BF16 && M % kMmaKC == 0 &&
           ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wg)) & 15) == 0)
    rc = dispatch_gate_mma(E, x, wg, logit_bias, T, M, k, normalize_gate, scores, idx, gates, w, st);
  else if (dtype == MOLE_BF16)     // odd M or unaligned rows: CUDA-core gate
    rc = dispatch_gate<__nv_bfloat16>(E, x, wg, logit_bias, T, M, k, normalize_gate, scores, idx, gates, w, st);
  else
    return fail(MOLE_ERR_UNSUPPORTED, "dtype %d", dtype);
  if (rc) return rc;
  return route_tail(w, T, E, k, C, idx, slot, gates, counts, offsets, perm, first_hist, l_aux, st);
}

}  // namespace mole

using namespace mole;

extern "C" int mole_route_workspace_bytes(int64_t T, int32_t E, int32_t k, int64_t* bytes) {
  MOLE_REQUIRE(bytes != nullptr, "bytes is null");
  if (int rc = check_route_args(T, E, k, 1)) return rc;
  *bytes = route_ws_bytes(T, E, k);
  return MOLE_OK;
}

extern "C" int mole_gate_route_fwd(const void* x, const void* wg, const float* logit_bias,
                                   int64_t T, int32_t M, int32_t E, int32_t k, int32_t C,
                                   int32_t normalize_gate, int32_t dtype, float* scores,
                                   int32_t* idx, int32_t* slot, float* gates, int32_t* counts,
                                   int32_t* offsets, int32_t* perm, int32_t* first_hist,
                                   float* l_aux, void* workspace, int64_t workspace_bytes,
                                   void* stream) {
  if (int rc = check_route_args(T, E, k, C)) return rc;
  MOLE_REQUIRE(x && wg && scores && idx && slot && gates && counts && offsets && perm &&
               first_hist && l_aux && workspace, "null pointer argument");
  MOLE_REQUIRE(M >= 1, "M=%d", M);
  MOLE_REQUIRE(workspace_bytes >= route_ws_bytes(T, E, k), "workspace too small: %lld < %lld",
               (long long)workspace_bytes, (long long)route_ws_bytes(T, E, k));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RouteWs w = carve(workspace, T, E, k);
  return gate_route_on(w, x, wg, logit_bias, T, M, E, k, C, normalize_gate, dtype, scores, idx, slot,
                       gates, counts, offsets, perm, first_hist, l_aux, st);
}

// ---- the same gate + routing build for callers that cannot hand over a workspace -------------
// The histogram / score-sum scratch lives in this fixed array inside the library's device image:
// every GPU that loads the library holds these 4 MiB until the process exits.
constexpr int64_t kStaticScratchBytes = 4 << 20;
static __device__ __align__(256) unsigned char g_route_scratch[kStaticScratchBytes];

// `g_route_scratch` in host code is only a handle for the runtime, not a device address: the
// address each device gave the array is looked up once per device (with that device current)
// and cached.
static int static_scratch(void** out) {
  static void* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  MOLE_CUDA_OK(cudaGetDevice(&dev));
  MOLE_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    MOLE_CUDA_OK(cudaGetSymbolAddress(&p, g_route_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return MOLE_OK;
}

extern "C" int mole_gate_route_fwd_static(const void* x, const void* wg, const float* logit_bias,
                                          int64_t T, int32_t M, int32_t E, int32_t k, int32_t C,
                                          int32_t normalize_gate, int32_t dtype, float* scores,
                                          int32_t* idx, int32_t* slot, float* gates,
                                          int32_t* counts, int32_t* offsets, int32_t* perm,
                                          int32_t* first_hist, float* l_aux, void* stream) {
  if (int rc = check_route_args(T, E, k, C)) return rc;
  MOLE_REQUIRE(x && wg && scores && idx && slot && gates && counts && offsets && perm &&
               first_hist && l_aux, "null pointer argument");
  MOLE_REQUIRE(M >= 1, "M=%d", M);
  const int64_t need = route_ws_bytes(T, E, k);
  if (need > kStaticScratchBytes)
    return fail(MOLE_ERR_UNSUPPORTED,
                "T=%lld tokens x E=%d experts x top-%d needs %lld bytes of routing scratch, the "
                "built-in scratch holds %lld: use mole_gate_route_fwd with a caller workspace",
                (long long)T, E, k, (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every scratch entry the scan reads is written by the gate kernel of this call first, so
  // nothing has to be cleared although the array keeps the previous call's contents
  RouteWs w = carve(scratch, T, E, k);
  return gate_route_on(w, x, wg, logit_bias, T, M, E, k, C, normalize_gate, dtype, scores, idx, slot,
                       gates, counts, offsets, perm, first_hist, l_aux, st);
}

extern "C" int mole_route_from_scores(const float* scores, int64_t T, int32_t E, int32_t k,
                                      int32_t C, int32_t normalize_gate, int32_t* idx,
                                      int32_t* slot, float* gates, int32_t* counts,
                                      int32_t* offsets, int32_t* perm, int32_t* first_hist,
                                      float* l_aux, void* workspace, int64_t workspace_bytes,
                                      void* stream) {
  if (int rc = check_route_args(T, E, k, C)) return rc;
  MOLE_REQUIRE(scores && idx && slot && gates && counts && offsets && perm && first_hist &&
               l_aux && workspace, "null pointer argument");
  MOLE_REQUIRE(workspace_bytes >= route_ws_bytes(T, E, k), "workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RouteWs w = carve(workspace, T, E, k);
  const int nb = nblocks(T);
  const size_t smem = (size_t)kGateTok * (E + 1) * 4 + (size_t)k * E * 4;
  MOLE_CUDA_OK(cudaFuncSetAttribute(topk_from_scores_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_from_scores_kernel<<<nb, kGateThreads, smem, st>>>(scores, T, E, k, normalize_gate, idx,
                                                          gates, w.hist, w.me_part, nb);
  MOLE_LAUNCH_OK();
  return route_tail(w, T, E, k, C, idx, slot, gates, counts, offsets, perm, first_hist, l_aux, st);
}

extern "C" int mole_gate_bwd(const float* scores, const int32_t* idx, const int32_t* slot,
                             const float* dgates, const float* d_l_aux,
                             const int32_t* first_hist, int64_t T, int32_t E, int32_t k, int32_t C,
                             int32_t normalize_gate, float* dlogits, void* stream) {
  if (int rc = check_route_args(T, E, k, C)) return rc;
  MOLE_REQUIRE(scores && idx && slot && dgates && first_hist && dlogits, "null pointer argument");
  gate_bwd_kernel<<<(unsigned)((T + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      scores, idx, slot, dgates, d_l_aux, first_hist, T, E, k, C, normalize_gate, dlogits);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// Token chunks of the gate weight gradient: about two blocks per SM, at least 256 tokens each
// (multiples of 128), the same split for the CUDA-core and the mma.sync kernel.
static void wgrad_split(int64_t T, int M, int col_width, int* chunk, int* n_chunks) {
  const int col_blocks = (M + col_width - 1) / col_width;
  // chunks per column block so that all blocks fit one wave of two per SM (rounding up left a
  // second, nearly empty wave)
  int64_t want = 2 * sm_count() / col_blocks;
  if (want < 1) want = 1;
  int64_t c = ((T + want - 1) / want + kWgTok - 1) / kWgTok * kWgTok;
  if (c < 256) c = 256;
  *chunk = (int)c;
  *n_chunks = (int)((T + c - 1) / c);
}
static bool wgrad_uses_mma(const void* x, int M, int dtype) {
  return dtype == MOLE_BF16 && M % 128 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
}

template <typename T>
static int launch_wgrad(const float* dlogits, const void* x, int64_t Ttok, int M, int E, int chunk,
                        int n_chunks, float* partial, cudaStream_t st) {
  dim3 grid((M + kWgCols - 1) / kWgCols, (unsigned)n_chunks);
  const int ej = (E + 15) / 16;
  const T* xp = static_cast<const T*>(x);
  if (ej <= 1) gate_wgrad_kernel<T, 1><<<grid, 256, 0, st>>>(dlogits, xp, Ttok, M, E, chunk, partial);
  else if (ej <= 2) gate_wgrad_kernel<T, 2><<<grid, 256, 0, st>>>(dlogits, xp, Ttok, M, E, chunk, partial);
  else if (ej <= 4) gate_wgrad_kernel<T, 4><<<grid, 256, 0, st>>>(dlogits, xp, Ttok, M, E, chunk, partial);
  else if (ej <= 8) gate_wgrad_kernel<T, 8><<<grid, 256, 0, st>>>(dlogits, xp, Ttok, M, E, chunk, partial);
  else gate_wgrad_kernel<T, 16><<<grid, 256, 0, st>>>(dlogits, xp, Ttok, M, E, chunk, partial);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_gate_wgrad_workspace_bytes(int64_t T, int32_t M, int32_t E, int32_t dtype,
                                               int64_t* bytes) {
  MOLE_REQUIRE(bytes != nullptr, "bytes is null");
  if (int rc = check_route_args(T, E, 1, 1)) return rc;
  MOLE_REQUIRE(M >= 1, "M=%d", M);
  int chunk, n_chunks;
  // the larger of the two kernels' splits, so that the size does not depend on the alignment of x
  wgrad_split(T, M, kWgCols, &chunk, &n_chunks);
  int64_t n = n_chunks;
  if (dtype == MOLE_BF16 && M % 128 == 0) {
    wgrad_split(T, M, 128, &chunk, &n_chunks);
    if (n_chunks > n) n = n_chunks;
  }
  *bytes = n * (int64_t)E * M * 4;
  return MOLE_OK;
}

extern "C" int mole_gate_wgrad(const float* dlogits, const void* x, int64_t T, int32_t M,
                               int32_t E, int32_t dtype, float* dwg32, void* workspace,
                               int64_t workspace_bytes, void* stream) {
  if (int rc = check_route_args(T, E, 1, 1)) return rc;
  MOLE_REQUIRE(dlogits && x && dwg32 && workspace, "null pointer argument");
  MOLE_REQUIRE(dtype == MOLE_F32 || dtype == MOLE_BF16, "dtype %d", dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool mma = wgrad_uses_mma(x, M, dtype);
  int chunk, n_chunks;
  wgrad_split(T, M, mma ? 128 : kWgCols, &chunk, &n_chunks);
  MOLE_REQUIRE(workspace_bytes >= (int64_t)n_chunks * E * M * 4, "workspace too small");
  float* partial = static_cast<float*>(workspace);
  int rc;
  if (mma) rc = launch_gate_wgrad_mma(dlogits, x, T, M, E, chunk, n_chunks, partial, st);
  else if (dtype == MOLE_F32) rc = launch_wgrad<float>(dlogits, x, T, M, E, chunk, n_chunks, partial, st);
  else rc = launch_wgrad<__nv_bfloat16>(dlogits, x, T, M, E, chunk, n_chunks, partial, st);
  if (rc) return rc;
  const int64_t n = (int64_t)E * M;
  gate_wgrad_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, n_chunks, n, dwg32);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}
