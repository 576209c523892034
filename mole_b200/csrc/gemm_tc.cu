// (c) Grouped expert GEMM on the sm_100a tensor cores: tcgen05.mma with TMEM accumulators,
// operands staged in shared memory by TMA (no multicast), persistent CTAs, warp-specialised:
//
//   warp 0        TMA producer   (one lane): activation / weight tiles -> smem ring
//   warp 1        MMA issuer     (one lane): tcgen05.mma over the ring, double-buffered TMEM
//   warps 2..17   epilogue       TMEM -> registers -> fused epilogue -> global memory
//
// One kernel template covers the six GEMMs of the expert FFN (MOLE/cpp/core.cpp:350-353
// forward, :388-412 backward):
//
//   rows mode   out[r, n] = epi(sum_k A[r, k] W_e(k, n))     per scheduled 128-row tile
//      FC1   A = x   (K-major), W1_e as [N=F][K=M] (K-major)   epi: +b1, store x1 and act(x1)
//      FC2   A = h   (K-major), W2_e as [K=F][N=M] (N-major)   epi: +b2
//      dX2   A = dO  (K-major), W2_e as [N=F][K=M] (K-major)   epi: * act'(x1)
//      dX    A = dX1 (K-major), W1_e as [K=F][N=M] (N-major)   epi: store
//   wgrad mode  out_e[p, q] (+)= sum_{r in tiles of e} A[r, p] B[r, q]    (both operands MN-major)
//      dW2   A = h, B = dO;   dW1   A = dX1, B = x
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records a code in the
// library's fault word, stops waiting for the rest of its run, still frees its TMEM and exits.
#include <cuda.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "gemm.cuh"

namespace mole {

constexpr int kBM = 128;          // rows of one UMMA (cta_group::1)
constexpr int kBK = 64;           // K elements per stage = one 128-byte swizzle span of bf16
// Weight-gradient mode: K runs over an expert's rows, a stage holds kWBK of them.  (32-row stages
// in a ring twice as deep were measured: 19-33 % slower -- twice the TMA requests and stage
// hand-shakes per output tile; the weight-gradient launch is sensitive to both.)
constexpr int kWBK = 64;
constexpr int kUmmaK = 16;
constexpr int kEpiWarps = 16;
constexpr int kThreads = 32 * (2 + kEpiWarps);

enum TcMode : int { TC_ROWS = 0, TC_WGRAD = 1 };

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait; false when it gave up.  `abort_flag` lives in shared memory: once any wait of
// this CTA has run out, later waits return false at once.  A role that sees false leaves its
// work loop: it issues no further TMA load or MMA and stores nothing more, so an output that
// the accumulator never reached is not written (the fault word tells the host that the step's
// results are not to be used).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* fault, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const uint64_t t0 = globaltimer_ns();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > 2000000000ull) {     // 2 s
        *abort_flag = 1;
        atomicCAS(fault, 0, code);
        return false;
      }
    }
  }
  return true;
}
// After an abort: what this CTA has already issued (TMA loads into its shared memory, MMAs that
// read it) gets a bounded time to land before the CTA frees its TMEM and exits.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity, uint64_t deadline_ns) {
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity))
    if ((++polls & 0xff) == 0 && globaltimer_ns() > deadline_ns) return;
}
// Producer side of the drain: stage s of a ring of `stages` has been armed
// n_s = issued / stages + (s < issued % stages) times; the parity of its last phase is (n_s - 1) & 1.
__device__ __forceinline__ void drain_loads(uint32_t full0, int stages, uint32_t issued) {
  const uint64_t deadline = globaltimer_ns() + 200000000ull;      // 0.2 s for all of them
  for (int s = 0; s < stages; ++s) {
    const uint32_t n_s = issued / stages + ((uint32_t)s < issued % stages ? 1u : 0u);
    if (n_s > 0) mbar_drain(full0 + 8 * s, (n_s - 1) & 1u, deadline);
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, bf16 (layouts as documented for UMMA):
//   K-major  : rows of 128 B (64 K elements), 8-row groups 1024 B apart (SBO); LBO unused
//   MN-major : 64 MN elements (128 B) contiguous per K row, 8 K rows per 1024-byte group (SBO),
//              next 64 MN elements `lbo_bytes` further (LBO)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;      // descriptor version of sm_100
  d |= (uint64_t)2 << 61;      // SWIZZLE_128B
  return d;
}

// 32 bf16 = 64 bytes per thread, moved as two 32-byte vectors so that every request covers a
// whole 32-byte sector
__device__ __forceinline__ void ld_v8(const void* p, uint32_t (&w)[8]) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]),
                 "=r"(w[6]), "=r"(w[7]) : "l"(p));
}
__device__ __forceinline__ void st_v8(void* p, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
                 "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* p, float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t w[8];
    ld_v8(p + 16 * i, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[16 * i + 2 * j] = __uint_as_float(w[j] << 16);
      v[16 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
}
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* p, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      __nv_bfloat162 b = __floats2bfloat162_rn(v[16 * i + 2 * j], v[16 * i + 2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&b);
    }
    st_v8(p + 16 * i, w);
  }
}

// Exact-GELU pieces for the bf16 epilogues.  Phi(x) = 0.5 (1 + erf(x / sqrt 2)) through the
// rational-exponential form of erfc (Abramowitz & Stegun 7.1.26, |error| < 1.5e-7, far below a
// bf16 ulp): with z = |x| / sqrt 2 and t = 1 / (1 + p z),
//   erfc(z) = t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-z^2).
// exp(-z^2) = exp(-x^2 / 2) is also the Gaussian density's exponential, so value and derivative
// share one ex2 and one rcp.  The fp32 layer keeps erff (CUDA-core path).
// 1 / d for d in [1, 2^126): one MUFU.RCP (a division by the fast-math intrinsic adds range handling)
__device__ __forceinline__ float rcp_approx(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}
struct GeluParts { float cdf, e; };     // Phi(x) and exp(-x^2 / 2)
__device__ __forceinline__ GeluParts gelu_parts(float x) {
  const float ax = fabsf(x);
  const float t = rcp_approx(fmaf(0.3275911f * 0.70710678f, ax, 1.0f));
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * x * -0.72134752f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(t, poly, 1.421413741f);
  poly = fmaf(t, poly, -0.284496736f);
  poly = fmaf(t, poly, 0.254829592f);
  const float half_erfc = 0.5f * t * poly * e;          // 0.5 erfc(|x| / sqrt 2)
  GeluParts g;
  g.cdf = x >= 0.f ? 1.0f - half_erfc : half_erfc;
  g.e = e;
  return g;
}
__device__ __forceinline__ float fast_act_fwd(float x, int act) {
  if (act == MOLE_ACT_RELU) return fmaxf(x, 0.f);
  return x * gelu_parts(x).cdf;
}
__device__ __forceinline__ float fast_act_grad(float x, int act, int gelu_bwd) {
  if (act == MOLE_ACT_RELU) return x > 0.f ? 1.f : 0.f;
  if (gelu_bwd == MOLE_GELU_BWD_TANH) return gelu_tanh_grad(x);
  const GeluParts g = gelu_parts(x);
  return fmaf(x * 0.39894228f, g.e, g.cdf);
}

struct TcParams {
  // schedule
  const int32_t* n_tiles;
  const int32_t* expert_tile_start;
  const int32_t* tile_row0;
  const int32_t* tile_expert;
  const int32_t* tile_rows;           // valid rows per tile: the weight-gradient GEMM stops its K loop there
  const int32_t* expert_pair_start;   // 2-CTA kernel: prefix of ceil(tiles / 2) per expert
  const int32_t* rowmap;              // FC2 / dX: output row of every GEMM row (-1: none), or null
  void* peer_base[kMaxPeers];         // with rowmap: receive buffer of every source rank (peer_n > 0)
  int peer_n, peer_rank, peer_L, peer_Cs;
  int n_experts, e_begin;
  int N, K;                 // rows mode: output columns / reduction.  wgrad: Q / unused
  int P;                    // wgrad: output rows per expert
  int epi, act, gelu_bwd, accumulate;
  int panel_split;          // panel kernel: experts of more than 320 rows are cut into panels of <= 256 rows
  float* colsum_ws;         // panel kernel, dX2: partial column sums [expert][panel][4][N], or null
  int colsum_panels;        // panels per expert the partial sums are laid out for
  int colsum_tiles;         // 1: colsum_ws is laid out per row tile instead, [row0 / 128][4][N] (CTA-pair tile kernel)
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int32_t* fault;
  SlotMap slot;
  // gate-weighted combine fused into the FC2 epilogue (one-CTA kernel, one source rank):
  // row (e, s) belongs to pair perm[offsets[e] + s] = t * k + j; y[t] += gates[pair] * out
  const int32_t* c_perm;
  const int32_t* c_offsets;
  const int32_t* c_counts;
  const float* c_gates;
  __nv_bfloat16* c_y;          // null: no fused combine
  int c_k, c_Cs;
};

// y[0..7] (eight bf16 pairs = 16 columns) += v, as two 16-byte reductions at L2.  With k <= 2 a
// token's row receives at most two addends, whose sum does not depend on their order.
__device__ __forceinline__ void red_add_bf16x16(__nv_bfloat16* y, const uint32_t (&v)[8]) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(y), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(y + 8), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

struct WorkItem {
  int valid;
  int row0;       // rows mode: first row of the tile.  wgrad: p0
  int n0;         // first output column
  int el;         // expert index relative to e_begin
  int t0, t1;     // wgrad: tile range of the expert
};

// `start` is the kernel's shared-memory copy of expert_tile_start: shared memory takes nearly all
// of the SM's L1, so a chain of dependent global loads (the binary search) would cost an L2 round
// trip per step, per work item, on the critical path of every role.
template <int MODE, int BN>
__device__ __forceinline__ WorkItem decode_item(const TcParams& p, const int* start, int item) {
  WorkItem w;
  w.valid = 0;
  if (MODE == TC_ROWS) {
    const int nb = p.N / BN;
    const int total = start[p.n_experts] * nb;
    if (item >= total) return w;
    int lo = 0, hi = p.n_experts;            // last expert with tile_start * nb <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (start[mid] * nb <= item) lo = mid; else hi = mid;
    }
    const int s = start[lo], nt = start[lo + 1] - s;
    const int local = item - s * nb;
    const int tile = s + local % nt;
    w.valid = 1;
    w.el = lo;
    w.row0 = p.tile_row0[tile];
    w.n0 = (local / nt) * BN;
    w.t0 = w.t1 = 0;
  } else {
    const int pb = p.P / kBM, qb = p.N / BN;
    if (item >= p.n_experts * pb * qb) return w;
    w.valid = 1;
    w.el = item / (pb * qb);
    const int r = item - w.el * pb * qb;
    w.row0 = (r / qb) * kBM;
    w.n0 = (r % qb) * BN;
    w.t0 = start[w.el];
    w.t1 = start[w.el + 1];
  }
  return w;
}

// Epilogue of one thread's accumulator row: columns [c_begin, c_end) of the tile in steps of 32,
// TMEM -> registers -> fused epilogue -> global memory (64 contiguous bytes per step and output).
// Epilogue kind, activation and GELU-derivative flavour are compile-time here (the run-time
// switch sits outside the column loop): the FC1 and dX2 epilogues are issue-bound, every
// per-element branch shows up in the GEMM's time.
template <int ACT>
__device__ __forceinline__ float act_fwd_t(float x) {
  if (ACT == MOLE_ACT_RELU) return fmaxf(x, 0.f);
  return x * gelu_parts(x).cdf;
}
template <int ACT, int GBWD>
__device__ __forceinline__ float act_grad_t(float x) {
  if (ACT == MOLE_ACT_RELU) return x > 0.f ? 1.f : 0.f;
  if (GBWD == MOLE_GELU_BWD_TANH) return gelu_tanh_grad(x);
  const GeluParts g = gelu_parts(x);
  return fmaf(x * 0.39894228f, g.e, g.cdf);
}
__device__ __forceinline__ float bf16_round(float v) {
  return __uint_as_float((__float_as_uint(v) + 0x7fffu + ((__float_as_uint(v) >> 16) & 1u)) & 0xffff0000u);
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&b);
}
// Pairs of values on the packed fp32 instructions (fma / mul / add .f32x2): the FC1 and dX2
// epilogues are bound by instruction issue, and the pair forms do the same operations in the same
// order as the scalar code in about half the instructions (results are bit-identical).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_dup(float a) { return f2_pack(a, a); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// gelu_parts on two values: the same operations in the same order
struct GeluParts2 { uint64_t cdf, e; };
__device__ __forceinline__ GeluParts2 gelu_parts2(uint64_t x) {
  float x0, x1;
  f2_unpack(x, x0, x1);
  const uint64_t d = f2_fma(f2_dup(0.3275911f * 0.70710678f), x & 0x7fffffff7fffffffull, f2_dup(1.0f));
  float d0, d1;
  f2_unpack(d, d0, d1);
  const uint64_t t = f2_pack(rcp_approx(d0), rcp_approx(d1));
  float a0, a1, e0, e1;
  f2_unpack(f2_mul(f2_mul(x, x), f2_dup(-0.72134752f)), a0, a1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
  GeluParts2 g;
  g.e = f2_pack(e0, e1);
  // the factor 0.5 of 0.5 * t * poly * e sits in the coefficients (an exact scaling)
  uint64_t poly = f2_fma(t, f2_dup(0.5f * 1.061405429f), f2_dup(0.5f * -1.453152027f));
  poly = f2_fma(t, poly, f2_dup(0.5f * 1.421413741f));
  poly = f2_fma(t, poly, f2_dup(0.5f * -0.284496736f));
  poly = f2_fma(t, poly, f2_dup(0.5f * 0.254829592f));
  const uint64_t he = f2_mul(f2_mul(t, poly), g.e);                     // 0.5 erfc(|x| / sqrt 2)
  const uint64_t up = f2_fma(he, f2_dup(-1.0f), f2_dup(1.0f));          // 1 - he
  float h0, h1, u0, u1;
  f2_unpack(he, h0, h1);
  f2_unpack(up, u0, u1);
  g.cdf = f2_pack(x0 >= 0.f ? u0 : h0, x1 >= 0.f ? u1 : h1);
  return g;
}
template <int ACT>
__device__ __forceinline__ uint32_t act_fwd_pair(uint32_t xw) {          // bf16 pair -> bf16 pair
  const float lo = bf16_lo(xw), hi = bf16_hi(xw);
  if (ACT == MOLE_ACT_RELU) return pack_bf16(fmaxf(lo, 0.f), fmaxf(hi, 0.f));
  const uint64_t x = f2_pack(lo, hi);
  float o0, o1;
  f2_unpack(f2_mul(x, gelu_parts2(x).cdf), o0, o1);
  return pack_bf16(o0, o1);
}
template <int ACT, int GBWD>
__device__ __forceinline__ uint32_t act_bwd_pair(float v0, float v1, uint32_t xw) {   // v * act'(x)
  const float lo = bf16_lo(xw), hi = bf16_hi(xw);
  if (ACT == MOLE_ACT_RELU || GBWD == MOLE_GELU_BWD_TANH)
    return pack_bf16(v0 * act_grad_t<ACT, GBWD>(lo), v1 * act_grad_t<ACT, GBWD>(hi));
  const uint64_t x = f2_pack(lo, hi);
  const GeluParts2 g = gelu_parts2(x);
  const uint64_t d = f2_fma(f2_mul(x, f2_dup(0.39894228f)), g.e, g.cdf);
  float o0, o1;
  f2_unpack(f2_mul(f2_pack(v0, v1), d), o0, o1);
  return pack_bf16(o0, o1);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// The epilogue works in steps of 16 columns: one tcgen05.ld of 16 accumulator columns, the fused
// arithmetic, one 32-byte store per output and thread.  Sixteen epilogue warps (four per
// scheduler) share a tile: with eight, each warp issued once in ~6.5 cycles (TMEM and global
// load latency, MUFU results) and the FC1 / dX2 epilogues took three times as long as the main
// loop they should hide behind.  Global operands of the epilogue (pre-activation for dX2, old
// gradient for "+=") are all fetched before the wait for the accumulator, so their latency
// overlaps the main loop; the bias slice of the tile sits in a per-warp shared-memory strip
// filled at the same point.
constexpr int kEpiStep = 16;

// Scattered output rows that go to another GPU (push-style exchange): 16- or 32-byte stores
// of 32 different rows per instruction cross NVLink as 32 small packets, and FC2 / dX ran at a
// sixth of the link bandwidth.  The warp's 32 rows x (NSTEPS * 16) columns go through a 1 KB
// shared-memory strip in passes (as in epilogue_lines below); after a pass NSTEPS neighbouring
// lanes hold one row's NSTEPS * 32 contiguous bytes, and fetch that row's destination (each row
// has its own: rank, chunk, slot) from the lane that owns the row.
constexpr int kScatterStripBytes = 1024;
template <int NSTEPS>
__device__ __forceinline__ void scatter_lines(const uint32_t (&o)[NSTEPS][8], __nv_bfloat16* rowptr,
                                              bool valid, uint8_t* strip) {
  constexpr int kRowBytes = NSTEPS * 32;
  constexpr int kRows = kScatterStripBytes / kRowBytes;   // rows per pass
  constexpr int kPasses = 32 / kRows;
  constexpr int kMask = (2 * NSTEPS - 1) & 7;
  static_assert(kRows * NSTEPS == 32, "one 32-byte piece per lane and pass");
  const int lane = threadIdx.x & 31;
  const int wr = lane % kRows, wpass = lane / kRows;
  const int rr = lane / NSTEPS, ra = lane % NSTEPS;
  const uint64_t myptr = reinterpret_cast<uint64_t>(rowptr);
  __syncwarp();
#pragma unroll
  for (int j = 0; j < kPasses; ++j) {
    if (wpass == j) {
#pragma unroll
      for (int q = 0; q < NSTEPS; ++q)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint4*>(strip + wr * kRowBytes + (((2 * q + h) ^ (wr & kMask)) << 4)) =
              make_uint4(o[q][4 * h], o[q][4 * h + 1], o[q][4 * h + 2], o[q][4 * h + 3]);
    }
    __syncwarp();
    const int owner = kRows * j + rr;                      // lane whose row this lane stores
    const uint64_t dptr = __shfl_sync(0xffffffffu, myptr, owner);
    const int dvalid = __shfl_sync(0xffffffffu, (int)valid, owner);
    const uint8_t* row = strip + rr * kRowBytes;
    const uint4 lo = *reinterpret_cast<const uint4*>(row + (((2 * ra) ^ (rr & kMask)) << 4));
    const uint4 hi = *reinterpret_cast<const uint4*>(row + (((2 * ra + 1) ^ (rr & kMask)) << 4));
    if (dvalid) {
      char* d = reinterpret_cast<char*>(dptr) + 32 * ra;
      asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};"
                   ::"l"(d), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
      asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};"
                   ::"l"(d + 16), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
    }
    __syncwarp();
  }
}

template <int EPI, int ACT, int GBWD, bool HAS_BIAS, bool ACCUM, int NSTEPS>
__device__ __forceinline__ void epilogue_loop(const TcParams& p, uint32_t taddr, bool empty,
                                              bool valid, __nv_bfloat16* sout, int64_t obase,
                                              const float* bias_s, int c_begin,
                                              uint32_t (&pre)[NSTEPS][8], uint8_t* strip,
                                              __nv_bfloat16* yrow = nullptr, float gate = 0.f,
                                              float* cs_part = nullptr, uint16_t* cs_strip = nullptr) {
  const bool remote = (EPI == EPI_BIAS || EPI == EPI_STORE) && p.peer_n > 0;
  uint32_t keep[NSTEPS][8];       // remote rows: the whole slice first, then whole-line stores
  {
#pragma unroll
    for (int step = 0; step < NSTEPS; ++step) {
      const int c = c_begin + kEpiStep * step;
      uint32_t (&cur)[8] = pre[step];
      uint32_t r[16];
      if (!empty) {
        tmem_ld16(taddr + c, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0u;
      }
      uint32_t o[8];
      if (EPI == EPI_WGRAD) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
          if (ACCUM) { lo += bf16_lo(cur[i]); hi += bf16_hi(cur[i]); }
          o[i] = pack_bf16(lo, hi);
        }
        st_v8(p.out0 + obase + c, o);
      } else if (EPI == EPI_FC1) {
        uint32_t h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
          if (HAS_BIAS) {
            const float2 b = *reinterpret_cast<const float2*>(bias_s + (c - c_begin) + 2 * i);
            lo += b.x; hi += b.y;
          }
          // the saved pre-activation is bf16: the activation is taken of the rounded value so
          // that backward's act'(x1) and forward's act(x1) see the same x1
          o[i] = pack_bf16(lo, hi);
          h[i] = act_fwd_pair<ACT>(o[i]);
        }
        st_v8(p.out0 + obase + c, o);
        st_v8(p.out1 + obase + c, h);
      } else if (EPI == EPI_BIAS) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
          if (HAS_BIAS) {
            const float2 b = *reinterpret_cast<const float2*>(bias_s + (c - c_begin) + 2 * i);
            lo += b.x; hi += b.y;
          }
          o[i] = pack_bf16(lo, hi);
        }
        if (remote) {
#pragma unroll
          for (int i = 0; i < 8; ++i) keep[step][i] = o[i];
        } else if (valid) {
          st_v8(sout + obase + c, o);
        }
        if (yrow != nullptr) {       // fused combine: the stored (rounded) row times its gate weight
          uint32_t gv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) gv[i] = pack_bf16(gate * bf16_lo(o[i]), gate * bf16_hi(o[i]));
          red_add_bf16x16(yrow + c, gv);
        }
      } else if (EPI == EPI_DACT) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = act_bwd_pair<ACT, GBWD>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), cur[i]);
        st_v8(p.out0 + obase + c, o);
        if (cs_part != nullptr) {
          // Column sums of the warp's 32 rows (of the stored, rounded values) for these 16 columns:
          // through a [16 columns][32 rows] strip of bf16 (1 KB); lane l adds 16 rows of column l % 16, starting
          // at a row that differs from lane to lane (no bank conflicts), and the two halves meet
          // in one shuffle.  Lanes 0-15 store the sums: one partial per (row tile, warp, column).
          const int lane = threadIdx.x & 31;
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            cs_strip[(2 * i) * 32 + lane] = (uint16_t)(o[i] & 0xffffu);
            cs_strip[(2 * i + 1) * 32 + lane] = (uint16_t)(o[i] >> 16);
          }
          __syncwarp();
          const int col = lane & 15, half = lane >> 4;
          float sum = 0.f;
#pragma unroll
          for (int rr = 0; rr < 16; ++rr)
            sum += __uint_as_float((uint32_t)cs_strip[col * 32 + half * 16 + ((rr + col) & 15)] << 16);
          sum += __shfl_xor_sync(0xffffffffu, sum, 16);
          if (half == 0) cs_part[c + col] = sum;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        if (remote) {
#pragma unroll
          for (int i = 0; i < 8; ++i) keep[step][i] = o[i];
        } else if (valid) {
          st_v8(sout + obase + c, o);
        }
        if (yrow != nullptr) {
          uint32_t gv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) gv[i] = pack_bf16(gate * bf16_lo(o[i]), gate * bf16_hi(o[i]));
          red_add_bf16x16(yrow + c, gv);
        }
      }
    }
  }
  if ((EPI == EPI_BIAS || EPI == EPI_STORE) && remote)
    scatter_lines<NSTEPS>(keep, sout + obase + c_begin, valid, strip);
}

// Epilogue with whole-line stores.  After tcgen05.ld a thread holds 16 consecutive columns of ONE
// row, so a plain warp store writes 32 rows x 32 bytes: 32 separate L2 requests and 9 LSU
// wavefronts per instruction, and the weight-gradient GEMM, whose output is its main traffic,
// spent half of its L2 tag and LSU capacity on them.  Here the warp's 32 rows x (NSTEPS * 16)
// columns go through a 2 KB shared-memory strip in passes of 16 rows (NSTEPS = 4); after a pass,
// NSTEPS neighbouring lanes hold one row's NSTEPS * 32 contiguous bytes and the store
// instruction writes whole 128-byte lines.  16-byte chunks are XOR-swizzled with the row so that
// neither side has bank conflicts.  The next use of the strip (next tile) comes after the
// TMEM wait of that tile, a warp-wide instruction, which orders it behind this tile's reads.
constexpr int kStripBytes = 2048;
template <int NSTEPS>
__device__ __forceinline__ void epilogue_lines(__nv_bfloat16* out, int64_t warp_base, int ldo,
                                               uint32_t taddr, bool empty, int c_begin,
                                               uint8_t* strip) {
  constexpr int kRowBytes = NSTEPS * 32;
  constexpr int kRows = kStripBytes / kRowBytes;      // rows per pass
  constexpr int kPasses = 32 / kRows;
  constexpr int kPieces = kRows * NSTEPS / 32;        // 32-byte pieces a lane stores per pass
  constexpr int kMask = (2 * NSTEPS - 1) & 7;
  const int lane = threadIdx.x & 31;
  uint32_t o[NSTEPS][8];
#pragma unroll
  for (int q = 0; q < NSTEPS; ++q) {
    uint32_t r[16];
    if (!empty) {
      tmem_ld16(taddr + c_begin + kEpiStep * q, r);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = 0u;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o[q][i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
  }
  const int wr = lane % kRows, wpass = lane / kRows;      // as a writer of the strip
  __syncwarp();                                           // the previous tile's readers are done
#pragma unroll
  for (int j = 0; j < kPasses; ++j) {
    if (wpass == j) {
#pragma unroll
      for (int q = 0; q < NSTEPS; ++q)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint4*>(strip + wr * kRowBytes + (((2 * q + h) ^ (wr & kMask)) << 4)) =
              make_uint4(o[q][4 * h], o[q][4 * h + 1], o[q][4 * h + 2], o[q][4 * h + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < kPieces; ++k) {
      const int idx = lane + 32 * k;
      const int rr = idx / NSTEPS, ra = idx % NSTEPS;     // row of the pass, 32-byte piece of the row
      const uint8_t* row = strip + rr * kRowBytes;
      const uint4 lo = *reinterpret_cast<const uint4*>(row + (((2 * ra) ^ (rr & kMask)) << 4));
      const uint4 hi = *reinterpret_cast<const uint4*>(row + (((2 * ra + 1) ^ (rr & kMask)) << 4));
      const uint32_t v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      st_v8(out + warp_base + (int64_t)(kRows * j + rr) * ldo + c_begin + kEpiStep * ra, v);
    }
    if (j + 1 < kPasses) __syncwarp();
  }
}

// Epilogue variants.  Each kernel instantiation carries exactly one: a kernel that holds all of
// them behind a run-time switch is several times larger and misses in the instruction cache.
enum EpiVariant : int {
  EV_FC1_GELU_B, EV_FC1_GELU, EV_FC1_RELU_B, EV_FC1_RELU,     // FC1 with / without bias
  EV_DACT_GELU, EV_DACT_TANH, EV_DACT_RELU,                   // dX2
  EV_BIAS, EV_STORE,                                          // FC2 with bias / FC2 without, dX
  EV_WGRAD, EV_WGRAD_ACC
};
template <int EV> struct EvTraits {
  static constexpr int epi = EV <= EV_FC1_RELU ? EPI_FC1 : EV <= EV_DACT_RELU ? EPI_DACT
                             : EV == EV_BIAS ? EPI_BIAS : EV == EV_STORE ? EPI_STORE : EPI_WGRAD;
  static constexpr int act = (EV == EV_FC1_RELU_B || EV == EV_FC1_RELU || EV == EV_DACT_RELU)
                                 ? MOLE_ACT_RELU : MOLE_ACT_GELU;
  static constexpr int gbwd = EV == EV_DACT_TANH ? MOLE_GELU_BWD_TANH : MOLE_GELU_BWD_EXACT;
  static constexpr bool bias = EV == EV_FC1_GELU_B || EV == EV_FC1_RELU_B || EV == EV_BIAS;
  static constexpr bool accum = EV == EV_WGRAD_ACC;
  static constexpr bool prefetch = epi == EPI_DACT || accum;
  static constexpr bool scatter = epi == EPI_BIAS || epi == EPI_STORE;   // outputs that may be scattered
};

// Issued before the wait for the accumulator: the first two prefetch steps and the bias strip.
template <int EV, int NSTEPS>
__device__ __forceinline__ void epilogue_prefetch(const TcParams& p, int64_t obase,
                                                  const __nv_bfloat16* bias, float* bias_s,
                                                  int c_begin, uint32_t (&pre)[NSTEPS][8]) {
  if (EvTraits<EV>::prefetch) {
    const __nv_bfloat16* src = EvTraits<EV>::epi == EPI_WGRAD ? p.out0 : p.aux;
#pragma unroll
    for (int step = 0; step < NSTEPS; ++step) ld_v8(src + obase + c_begin + kEpiStep * step, pre[step]);
  }
  if (EvTraits<EV>::bias) {
    const int lane = threadIdx.x & 31;
    __syncwarp();                       // the strip's previous readers are done
    for (int i = lane; i < NSTEPS * kEpiStep; i += 32) bias_s[i] = __bfloat162float(bias[c_begin + i]);
    __syncwarp();
  }
}

template <int MODE, bool B_KMAJOR, int BN, int STAGES, int EV>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ TcParams p) {
  constexpr int KR = MODE == TC_WGRAD ? kWBK : kBK;       // K extent of one shared-memory stage
  constexpr uint32_t kBoxBytes = 128 * KR;                // one 64-element-wide MN-major TMA box
  constexpr uint32_t kABytes = kBM * KR * 2;
  constexpr uint32_t kBBytes = BN * KR * 2;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;     // two accumulator stages (256 or 512 columns)
  constexpr bool A_MN = (MODE == TC_WGRAD);
  constexpr bool B_MN = (MODE == TC_WGRAD) || !B_KMAJOR;
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                              ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                              ((uint32_t)(kBM >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 5];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag_s;
  __shared__ __align__(16) float bias_strip[kEpiWarps][64];       // per epilogue warp: bias of its columns
  __shared__ __align__(16) uint8_t store_strip[kEpiWarps][kStripBytes];   // per epilogue warp: epilogue_lines
  __shared__ __align__(16) uint8_t scatter_strip[kEpiWarps][kScatterStripBytes];   // ... scatter_lines
  __shared__ int start_s[kMaxLocalExperts + 1];                   // expert_tile_start, see decode_item
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
  const uint32_t drain0 = smem_u32(&bars[2 * STAGES + 4]);      // used only after an abort
  const uint32_t smem_base = smem_u32(smem);

  for (int i = threadIdx.x; i <= p.n_experts; i += kThreads) start_s[i] = p.expert_tile_start[i];
  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    mbar_init(drain0, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------
    // Rows mode: one lane issues the stage's loads (two large boxes with K-major weights).
    // Weight-gradient mode: a stage is six boxes of 8 KB (both operands MN-major, 64 columns per
    // box); the whole warp runs the loop and lanes 0..5 issue one box each, so the requests of a
    // stage leave together instead of one after the other from a single thread.
    if (MODE == TC_WGRAD || lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok; item += gridDim.x) {
        const WorkItem w = decode_item<MODE, BN>(p, start_s, item);
        if (!w.valid) break;
        const int slot = p.slot.s[p.e_begin + w.el];
        if (MODE == TC_ROWS) {
          const int nkb = p.K / kBK;
          for (int kb = 0; kb < nkb; ++kb) {
            if (!(ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.fault, 1))) break;
            const uint32_t bar = full0 + 8 * stage;
            const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + kABytes;
            mbar_expect_tx(bar, kStageBytes);
            tma_load_2d(sa, &tmap_a, bar, kb * kBK, w.row0);
            if (B_KMAJOR) {
              tma_load_3d(sb, &tmap_b, bar, kb * kBK, w.n0, slot);
            } else {
#pragma unroll
              for (int i = 0; i < BN / 64; ++i)
                tma_load_3d(sb + i * kBoxBytes, &tmap_b, bar, w.n0 + 64 * i, kb * kBK, slot);
            }
            ++issued;
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        } else {
          // K runs over the expert's rows, tile by tile, and stops at each tile's valid rows
          // (64-row blocks here, 16-row MMA steps in the issuer): with ~256 rows per expert the
          // zero rows up to the next multiple of 128 would be a fifth of the work.
          constexpr int kBoxesA = kBM / 64, kBoxes = kBoxesA + BN / 64;
          for (int t = w.t0; t < w.t1 && ok; ++t) {
            const int trow = p.tile_row0[t];
            const int halves = (p.tile_rows[t] + KR - 1) / KR;
            for (int hf = 0; hf < halves; ++hf) {
              // every lane waits (the same barrier, the same answer up to the moment of a time-out)
              ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.fault, 1));
              if (!ok) break;
              const uint32_t bar = full0 + 8 * stage;
              const uint32_t sa = smem_base + stage * kStageBytes;
              const int row = trow + hf * KR;
              if (lane == 0) mbar_expect_tx(bar, kStageBytes);
              __syncwarp();                   // the expectation is armed before any box can complete
              if (lane < kBoxesA)
                tma_load_2d(sa + lane * kBoxBytes, &tmap_a, bar, w.row0 + 64 * lane, row);
              else if (lane < kBoxes)
                tma_load_2d(sa + lane * kBoxBytes, &tmap_b, bar, w.n0 + 64 * (lane - kBoxesA), row);
              ++issued;
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
      if (lane == 0 && *abort_flag) drain_loads(full0, STAGES, issued);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok; item += gridDim.x) {
        const WorkItem w = decode_item<MODE, BN>(p, start_s, item);
        if (!w.valid) break;
        if (MODE == TC_WGRAD && w.t1 == w.t0) continue;      // empty expert: epilogue writes zeros
        if (!(ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.fault, 2))) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // one shared-memory stage: `ksteps` MMAs of K = 16
        auto issue_stage = [&](int ksteps, bool first) {
          if (!ok || !(ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.fault, 3))) return;
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + kABytes;
          auto mma_step = [&](int ks) {
            const uint64_t ad = A_MN ? make_desc(sa + ks * (kUmmaK * 128), kBoxBytes, 1024)
                                     : make_desc(sa + ks * (kUmmaK * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_desc(sb + ks * (kUmmaK * 128), kBoxBytes, 1024)
                                     : make_desc(sb + ks * (kUmmaK * 2), 16, 1024);
            tcgen05_mma_bf16(d_tmem, ad, bd, kIdesc, (first && ks == 0) ? 0u : 1u);
          };
          // a full stage is straight-line code: a branch between the MMAs of a stage slows their
          // issue (measured: the same MMAs behind a run-time condition each took 30 % longer)
          if (ksteps == KR / kUmmaK) {
#pragma unroll
            for (int ks = 0; ks < KR / kUmmaK; ++ks) mma_step(ks);
          } else {
            for (int ks = 0; ks < ksteps; ++ks) mma_step(ks);
          }
          tcgen05_commit(empty0 + 8 * stage);         // frees the smem stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        };
        if (MODE == TC_ROWS) {
          const int nkb = p.K / kBK;
          for (int kb = 0; kb < nkb; ++kb) issue_stage(kBK / kUmmaK, kb == 0);
        } else {
          bool first = true;
          for (int t = w.t0; t < w.t1; ++t) {
            const int v = p.tile_rows[t];
            const int halves = (v + KR - 1) / KR;
            for (int hf = 0; hf < halves; ++hf) {
              const int left = v - hf * KR;
              issue_stage(left >= KR ? KR / kUmmaK : (left + kUmmaK - 1) / kUmmaK, first);
              first = false;
            }
          }
        }
        if (!ok) break;                               // gave up: this accumulator is never published
        tcgen05_commit(tfull0 + 8 * acc);             // accumulator ready for the epilogue
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (*abort_flag) {                              // MMAs already issued retire before the TMEM goes
        tcgen05_commit(drain0);
        mbar_drain(drain0, 0, globaltimer_ns() + 200000000ull);
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;                     // TMEM lanes this warp may read
    const int cq = ew >> 2;                           // which quarter of the BN columns
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int item = blockIdx.x;; item += gridDim.x) {
      const WorkItem w = decode_item<MODE, BN>(p, start_s, item);
      if (!w.valid) break;
      const int e = p.e_begin + w.el;
      const int slot = p.slot.s[e];
      const bool empty = MODE == TC_WGRAD && w.t1 == w.t0;
      const int lrow = quarter * 32 + lane;
      int64_t obase;            // element offset of (row, n0) in the output
      bool valid = true;
      __nv_bfloat16* sout = p.out0;     // where a scattered row goes (FC2 / dX)
      if (MODE == TC_ROWS) {
        int64_t orow = w.row0 + lrow;
        if (EvTraits<EV>::scatter && p.rowmap != nullptr) {
          orow = p.rowmap[orow];
          valid = orow >= 0;
          if (p.peer_n > 0 && valid) {          // row of chunk [w][l] -> source rank w's buffer
            const int per_rank = p.peer_L * p.peer_Cs;
            const int wq = (int)(orow / per_rank);
            const int rem = (int)(orow - (int64_t)wq * per_rank);
            const int l = rem / p.peer_Cs;
            sout = static_cast<__nv_bfloat16*>(p.peer_base[wq]);
            orow = ((int64_t)p.peer_rank * p.peer_L + l) * p.peer_Cs + (rem - l * p.peer_Cs);
          }
        }
        obase = orow * p.N + w.n0;
      } else {
        obase = ((int64_t)slot * p.P + w.row0 + lrow) * p.N + w.n0;
      }
      const __nv_bfloat16* bias =
          (MODE == TC_ROWS && p.bias) ? p.bias + (int64_t)slot * p.N + w.n0 : nullptr;
      constexpr int NSTEPS = BN / 4 / kEpiStep;
      uint32_t pre[NSTEPS][8];
      // fused combine (FC2, rows not scattered): where this thread's row goes, with which gate weight
      __nv_bfloat16* yrow = nullptr;
      float gate = 0.f;
      if (MODE == TC_ROWS && EvTraits<EV>::scatter && p.c_y != nullptr) {
        const int srow = w.row0 + lrow - e * p.c_Cs;
        if (srow < p.c_counts[e]) {
          const int pair = p.c_perm[p.c_offsets[e] + srow];
          gate = p.c_gates[pair];
          yrow = p.c_y + (int64_t)(pair / p.c_k) * p.N + w.n0;
        }
      }
      epilogue_prefetch<EV, NSTEPS>(p, obase, bias, bias_strip[ew], cq * (BN / 4), pre);
      if (!empty) {
        // warp-uniform: the epilogue's tcgen05.ld and shuffles need all 32 lanes
        if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.fault, 4)))
          break;                                      // nothing is stored for this tile
        tcgen05_fence_after();
      }
      using Ev = EvTraits<EV>;
      if (EV == EV_WGRAD)
        epilogue_lines<NSTEPS>(p.out0, obase - (int64_t)lane * p.N, p.N,
                               tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, empty,
                               cq * (BN / 4), store_strip[ew]);
      else
        epilogue_loop<Ev::epi, Ev::act, Ev::gbwd, Ev::bias, Ev::accum, NSTEPS>(
            p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, empty, valid, sout, obase,
            bias_strip[ew], cq * (BN / 4), pre, scatter_strip[ew], yrow, gate);
      if (!empty) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols) : "memory");
  }
}

// =========================================================================================
// cta_group::2 variant: a pair of CTAs on two SMs (a cluster of 2) computes a 256 x 256 tile.
// Each CTA stages its own 128 rows of A and one 128-column half of B; one tcgen05.mma issued by
// the even CTA reads A and both halves of B from both CTAs' shared memory and writes 128 lanes
// x 256 columns of accumulator into each CTA's TMEM.  Per unit of work the operand bytes read
// through L2 drop from 48 KB to 32 KB per 128 x 256 x 64 block-product -- the grouped GEMMs with
// few rows per expert are bound by L2 throughput, not by HBM or the tensor pipe.
//
//   rows mode   the pair takes two consecutive row tiles of one expert (the odd CTA idles its A
//               loads and its epilogue when the expert has an odd number of tiles)
//   wgrad mode  the pair takes a 256 x 256 block of the expert's [F, M] gradient
//
// Barriers: TMA loads of both CTAs complete on the even CTA's "full" barrier (.cta_group::2
// form, no multicast); stage release and accumulator-ready are tcgen05.commit arrivals multicast
// to both CTAs' barriers; the odd CTA's epilogue releases the accumulator with a remote arrive.
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;     // clears the CTA-rank bit of a shared::cluster address
constexpr int kBN2 = 256;
template <int KR> struct Pair2 {
  static constexpr uint32_t kBoxBytes = 128 * KR;
  static constexpr uint32_t kABytes = kBM * KR * 2;
  static constexpr uint32_t kBHalfBytes = (kBN2 / 2) * KR * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBHalfBytes;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                             int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                             int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tcgen05_commit2(uint32_t bar) {   // arrives in both CTAs of the pair
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tcgen05_mma2_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

struct PairItem {
  int valid;
  int el;
  int n0;          // first output column of the pair's 256-wide block
  int row0[2];     // rows mode: first row of each CTA's tile, -1 = none.  wgrad: p0 of each CTA
  int t0, t1;      // wgrad: tile range of the expert
};

template <int MODE>
__device__ __forceinline__ PairItem decode_pair(const TcParams& p, const int* start, const int* pstart, int item) {
  PairItem w;
  w.valid = 0;
  if (MODE == TC_ROWS) {
    const int nb = p.N / kBN2;
    const int total = pstart[p.n_experts] * nb;
    if (item >= total) return w;
    int lo = 0, hi = p.n_experts;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (pstart[mid] * nb <= item) lo = mid; else hi = mid;
    }
    const int ps = pstart[lo], np = pstart[lo + 1] - ps;
    const int local = item - ps * nb;
    const int pair = local % np;
    const int ts = start[lo], te = start[lo + 1];
    w.valid = 1;
    w.el = lo;
    w.n0 = (local / np) * kBN2;
    w.row0[0] = p.tile_row0[ts + 2 * pair];
    w.row0[1] = ts + 2 * pair + 1 < te ? p.tile_row0[ts + 2 * pair + 1] : -1;
    w.t0 = w.t1 = 0;
  } else {
    const int pb = p.P / 256, qb = p.N / kBN2;
    if (item >= p.n_experts * pb * qb) return w;
    w.valid = 1;
    w.el = item / (pb * qb);
    const int r = item - w.el * pb * qb;
    w.row0[0] = (r / qb) * 256;
    w.row0[1] = w.row0[0] + 128;
    w.n0 = (r % qb) * kBN2;
    w.t0 = start[w.el];
    w.t1 = start[w.el + 1];
  }
  return w;
}

template <int MODE, bool B_KMAJOR, int STAGES, int EV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tc2_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ TcParams p) {
  constexpr uint32_t kTmemCols = 2 * kBN2;
  constexpr int KR = MODE == TC_WGRAD ? kWBK : kBK;
  constexpr uint32_t kBoxBytes = Pair2<KR>::kBoxBytes;
  constexpr uint32_t kABytes = Pair2<KR>::kABytes;
  constexpr uint32_t kBHalfBytes = Pair2<KR>::kBHalfBytes;
  constexpr uint32_t kStage2Bytes = Pair2<KR>::kStageBytes;
  constexpr bool A_MN = (MODE == TC_WGRAD);
  constexpr bool B_MN = (MODE == TC_WGRAD) || !B_KMAJOR;
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                              ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(kBN2 >> 3) << 17) |
                              ((uint32_t)(256 >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 5];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag_s;
  __shared__ __align__(16) float bias_strip[kEpiWarps][64];       // per epilogue warp: bias of its columns
  __shared__ __align__(16) uint8_t store_strip[kEpiWarps][kStripBytes];   // per epilogue warp: epilogue_lines
  __shared__ __align__(16) uint8_t scatter_strip[kEpiWarps][kScatterStripBytes];   // ... scatter_lines
  __shared__ int start_s[kMaxLocalExperts + 1], pstart_s[kMaxLocalExperts + 1];    // see decode_item
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
  const uint32_t drain0 = smem_u32(&bars[2 * STAGES + 4]);      // used only after an abort
  const uint32_t smem_base = smem_u32(smem);
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  for (int i = threadIdx.x; i <= p.n_experts; i += kThreads) {
    start_s[i] = p.expert_tile_start[i];
    pstart_s[i] = p.expert_pair_start[i];
  }
  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    mbar_init(drain0, 1);          // the drain commit is multicast like the others: one arrival per CTA
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);               // the even CTA's arrive.expect_tx
      mbar_init(empty0 + 8 * s, 1);              // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 2 * kEpiWarps); // epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  cluster_sync_all();                            // peer barriers initialised, TMEM address published
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued = 0;
      bool ok = true;
      for (int item = cluster_id; ok; item += n_clusters) {
        const PairItem w = decode_pair<MODE>(p, start_s, pstart_s, item);
        if (!w.valid) break;
        const int slot = p.slot.s[p.e_begin + w.el];
        const bool have_a = w.row0[rank] >= 0;
        const uint32_t tx = MODE == TC_ROWS
                                ? kABytes * (w.row0[1] >= 0 ? 2u : 1u) + 2u * kBHalfBytes
                                : 2u * kStage2Bytes;
        const int nh = w.n0 + 128 * (int)rank;         // this CTA's half of the B columns
        if (MODE == TC_ROWS) {
          const int nkb = p.K / kBK;
          for (int kb = 0; kb < nkb; ++kb) {
            if (!(ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.fault, 11))) break;
            const uint32_t bar = (full0 + 8 * stage) & kPeerMask;     // the even CTA's barrier
            const uint32_t sa = smem_base + stage * kStage2Bytes, sb = sa + kABytes;
            if (leader) mbar_expect_tx(full0 + 8 * stage, tx);
            if (have_a) tma2_load_2d(sa, &tmap_a, bar, kb * kBK, w.row0[rank]);
            if (B_KMAJOR) {
              tma2_load_3d(sb, &tmap_b, bar, kb * kBK, nh, slot);
            } else {
#pragma unroll
              for (int i = 0; i < 2; ++i)
                tma2_load_3d(sb + i * kBoxBytes, &tmap_b, bar, nh + 64 * i, kb * kBK, slot);
            }
            ++issued;
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        } else {
          for (int t = w.t0; t < w.t1 && ok; ++t) {      // K stops at each tile's valid rows
            const int trow = p.tile_row0[t];
            const int halves = (p.tile_rows[t] + KR - 1) / KR;
            for (int hf = 0; hf < halves; ++hf) {
              if (!(ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.fault, 11))) break;
              const uint32_t bar = (full0 + 8 * stage) & kPeerMask;
              const uint32_t sa = smem_base + stage * kStage2Bytes, sb = sa + kABytes;
              const int row = trow + hf * KR;
              if (leader) mbar_expect_tx(full0 + 8 * stage, tx);
#pragma unroll
              for (int i = 0; i < 2; ++i)
                tma2_load_2d(sa + i * kBoxBytes, &tmap_a, bar, w.row0[rank] + 64 * i, row);
#pragma unroll
              for (int i = 0; i < 2; ++i)
                tma2_load_2d(sb + i * kBoxBytes, &tmap_b, bar, nh + 64 * i, row);
              ++issued;
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
      // both CTAs' loads complete on the even CTA's barriers: it waits for the pair (the odd CTA
      // stays until the cluster barrier at the end, which the even CTA reaches after this)
      if (leader && *abort_flag) drain_loads(full0, STAGES, issued);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA only) -----------------------
    if (lane == 0 && leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = cluster_id; ok; item += n_clusters) {
        const PairItem w = decode_pair<MODE>(p, start_s, pstart_s, item);
        if (!w.valid) break;
        if (MODE == TC_WGRAD && w.t1 == w.t0) continue;
        if (!(ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.fault, 12))) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN2;
        auto issue_stage = [&](int ksteps, bool first) {
          if (!ok || !(ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.fault, 13))) return;
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kStage2Bytes, sb = sa + kABytes;
          auto mma_step = [&](int ks) {
            const uint64_t ad = A_MN ? make_desc(sa + ks * (kUmmaK * 128), kBoxBytes, 1024)
                                     : make_desc(sa + ks * (kUmmaK * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_desc(sb + ks * (kUmmaK * 128), kBoxBytes, 1024)
                                     : make_desc(sb + ks * (kUmmaK * 2), 16, 1024);
            tcgen05_mma2_bf16(d_tmem, ad, bd, kIdesc, (first && ks == 0) ? 0u : 1u);
          };
          if (ksteps == KR / kUmmaK) {                // straight-line, see tc_gemm_kernel
#pragma unroll
            for (int ks = 0; ks < KR / kUmmaK; ++ks) mma_step(ks);
          } else {
            for (int ks = 0; ks < ksteps; ++ks) mma_step(ks);
          }
          tcgen05_commit2(empty0 + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        };
        if (MODE == TC_ROWS) {
          const int nkb = p.K / kBK;
          for (int kb = 0; kb < nkb; ++kb) issue_stage(kBK / kUmmaK, kb == 0);
        } else {
          bool first = true;
          for (int t = w.t0; t < w.t1; ++t) {
            const int v = p.tile_rows[t];
            const int halves = (v + KR - 1) / KR;
            for (int hf = 0; hf < halves; ++hf) {
              const int left = v - hf * KR;
              issue_stage(left >= KR ? KR / kUmmaK : (left + kUmmaK - 1) / kUmmaK, first);
              first = false;
            }
          }
        }
        if (!ok) break;
        tcgen05_commit2(tfull0 + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (*abort_flag) {                      // MMAs already issued retire before the TMEM goes
        tcgen05_commit2(drain0);
        mbar_drain(drain0, 0, globaltimer_ns() + 200000000ull);
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -----------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int cq = ew >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int item = cluster_id;; item += n_clusters) {
      const PairItem w = decode_pair<MODE>(p, start_s, pstart_s, item);
      if (!w.valid) break;
      const int slot = p.slot.s[p.e_begin + w.el];
      const bool empty = MODE == TC_WGRAD && w.t1 == w.t0;
      const int lrow = quarter * 32 + lane;
      const int r0 = w.row0[rank];
      int64_t obase = 0;
      bool valid = true;
      __nv_bfloat16* sout = p.out0;
      const __nv_bfloat16* bias = nullptr;
      constexpr int NSTEPS = kBN2 / 4 / kEpiStep;
      uint32_t pre[NSTEPS][8];
      if (r0 >= 0) {
        if (MODE == TC_ROWS) {
          int64_t orow = r0 + lrow;
          if (EvTraits<EV>::scatter && p.rowmap != nullptr) {
            orow = p.rowmap[orow];
            valid = orow >= 0;
            if (p.peer_n > 0 && valid) {
              const int per_rank = p.peer_L * p.peer_Cs;
              const int wq = (int)(orow / per_rank);
              const int rem = (int)(orow - (int64_t)wq * per_rank);
              const int l = rem / p.peer_Cs;
              sout = static_cast<__nv_bfloat16*>(p.peer_base[wq]);
              orow = ((int64_t)p.peer_rank * p.peer_L + l) * p.peer_Cs + (rem - l * p.peer_Cs);
            }
          }
          obase = orow * p.N + w.n0;
        } else {
          obase = ((int64_t)slot * p.P + r0 + lrow) * p.N + w.n0;
        }
        bias = (MODE == TC_ROWS && p.bias) ? p.bias + (int64_t)slot * p.N + w.n0 : nullptr;
        epilogue_prefetch<EV, NSTEPS>(p, obase, bias, bias_strip[ew], cq * (kBN2 / 4), pre);
      }
      if (!empty) {
        if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.fault, 14)))
          break;                                      // nothing is stored for this tile
        tcgen05_fence_after();
      }
      if (r0 >= 0)
      {
        using Ev = EvTraits<EV>;
        if (EV == EV_WGRAD)
          epilogue_lines<NSTEPS>(p.out0, obase - (int64_t)lane * p.N, p.N,
                                 tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN2, empty,
                                 cq * (kBN2 / 4), store_strip[ew]);
        else {
          // dX2 with fused column sums: this warp's partial row for its (row tile, quarter)
          float* cs_part = nullptr;
          if (Ev::epi == EPI_DACT && MODE == TC_ROWS && p.colsum_ws != nullptr && p.colsum_tiles)
            cs_part = p.colsum_ws + ((int64_t)(r0 / kTileRows) * 4 + quarter) * p.N + w.n0;
          epilogue_loop<Ev::epi, Ev::act, Ev::gbwd, Ev::bias, Ev::accum, NSTEPS>(
              p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN2, empty, valid, sout, obase,
              bias_strip[ew], cq * (kBN2 / 4), pre, scatter_strip[ew], nullptr, 0.f, cs_part,
              reinterpret_cast<uint16_t*>(scatter_strip[ew]));
        }
      }
      if (!empty) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster((tempty0 + 8 * acc) & kPeerMask);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  }

  tcgen05_fence_before();
  cluster_sync_all();          // nobody leaves while the peer may still touch its smem or barriers
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols) : "memory");
  }
}

#include "gemm_panel.cuh"

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Encoded tensor maps are cached by (base, extents, box): a training loop presents the same few
// buffers every step and the driver call costs microseconds on the launch path.
struct MapKey {
  uintptr_t base;
  uint64_t d[3];
  uint32_t b[3];
  int rank;
  bool operator==(const MapKey& o) const {
    return base == o.base && rank == o.rank && d[0] == o.d[0] && d[1] == o.d[1] && d[2] == o.d[2] &&
           b[0] == o.b[0] && b[1] == o.b[1] && b[2] == o.b[2];
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 3; ++i) h = (h ^ (k.d[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2))) * 31 + k.b[i];
    return (size_t)(h ^ (uint64_t)k.rank);
  }
};
static int encode_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                      const uint32_t* box);
static int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                    const uint32_t* box) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{};
  key.base = reinterpret_cast<uintptr_t>(base);
  key.rank = rank;
  for (int i = 0; i < rank; ++i) { key.d[i] = dims[i]; key.b[i] = box[i]; }
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *m = it->second; return MOLE_OK; }
  if (int rc = encode_map(m, base, rank, dims, box)) return rc;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *m);
  return MOLE_OK;
}

// bf16 tensor, innermost dimension contiguous, 128-byte swizzle, box inner extent 64 elements
static int encode_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                      const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MOLE_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t gdim[3], gstride[2];
  cuuint32_t bdim[3], estr[3] = {1, 1, 1};
  uint64_t stride = 2;
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    stride *= dims[i];
    if (i < rank - 1) gstride[i] = stride;
  }
  MOLE_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base %p not 16-byte aligned", base);
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim,
                        gstride, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOLE_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return MOLE_OK;
}

bool tc_supported(int M, int F) { return M % 128 == 0 && F % 128 == 0 && M >= 128 && F >= 128; }

template <int MODE, bool B_KMAJOR, int BN, int EV>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int max_items,
                     cudaStream_t st) {
  constexpr int KR = MODE == TC_WGRAD ? kWBK : kBK;
  constexpr int STAGES = (BN == 256 ? 4 : 6) * (kBK / KR);      // the same bytes in flight either way
  constexpr size_t smem = (size_t)STAGES * (kBM * KR * 2 + BN * KR * 2) + 1024;
  auto kern = tc_gemm_kernel<MODE, B_KMAJOR, BN, STAGES, EV>;
  static PerDeviceInt configured;          // the attribute belongs to a device
  const int dev = current_device();
  if (!configured.get(dev)) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.set(dev, 1);
  }
  int grid = sm_count();
  if (max_items < grid) grid = max_items;
  if (grid <= 0) return MOLE_OK;
  if (profile_enabled()) profile_begin(st, p.epi);
  kern<<<grid, kThreads, smem, st>>>(ma, mb, p);
  if (profile_enabled()) profile_end(st);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// Launch of the cta_group::2 kernel: grid = 2 x min(work units, clusters that can be resident).
template <int MODE, bool B_KMAJOR, int EV>
static int launch_tc2(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int max_items,
                      cudaStream_t st) {
  constexpr int KR = MODE == TC_WGRAD ? kWBK : kBK;
  constexpr int STAGES = 6 * (kBK / KR);
  constexpr size_t smem = (size_t)STAGES * Pair2<KR>::kStageBytes + 1024;
  auto kern = tc2_gemm_kernel<MODE, B_KMAJOR, STAGES, EV>;
  static PerDeviceInt max_clusters_of;     // attribute and occupancy belong to a device
  const int dev = current_device();
  int max_clusters = (int)max_clusters_of.get(dev);
  if (max_clusters == 0) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n;
    max_clusters_of.set(dev, n);
  }
  int clusters = max_clusters < max_items ? max_clusters : max_items;
  if (clusters <= 0) return MOLE_OK;
  if (profile_enabled()) profile_begin(st, p.epi);
  kern<<<2 * clusters, kThreads, smem, st>>>(ma, mb, p);
  if (profile_enabled()) profile_end(st);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// Launch of the panel kernel: as launch_tc2, one work unit = (expert, 256 features, row panel).
// `max_rows` bounds an expert's rows: it sizes the row area of a shared-memory stage.
template <bool W_KMAJOR, int EV>
static int launch_panel(const PanelMaps& maps, const TcParams& p, int max_items, int max_rows,
                        cudaStream_t st) {
  if (p.panel_split && max_rows > 320) max_rows = 320;      // no panel holds more
  const int n_max = max_rows > 512 ? 512 : (max_rows <= 256 ? ((max_rows + 15) & ~15) : ((max_rows + 31) & ~31));
  const uint32_t stage_bytes = kPanelABytes + (uint32_t)(n_max / 2) * 128u;
  // + the kernel's static 3.5 KB (and the 16 KB of transposing strips of the FC1 / dX2 epilogues):
  // under the 227 KB a block may have
  constexpr size_t kBudget = (panel_heavy(EvTraits<EV>::epi) ? 206 : 222) * 1024;
  int stages = (int)((kBudget - 1024) / stage_bytes);
  if (stages > kPanelMaxStages) stages = kPanelMaxStages;
  const size_t smem = (size_t)stages * stage_bytes + 1024;
  auto kern = panel_gemm_kernel<W_KMAJOR, EV>;
  static PerDeviceInt max_clusters_of;
  const int dev = current_device();
  int max_clusters = (int)max_clusters_of.get(dev);
  if (max_clusters == 0) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBudget));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n;
    max_clusters_of.set(dev, n);
  }
  int clusters = max_clusters < max_items ? max_clusters : max_items;
  if (clusters <= 0) return MOLE_OK;
  if (profile_enabled()) profile_begin(st, p.epi);
  kern<<<2 * clusters, kThreads, smem, st>>>(maps, p, stages, stage_bytes);
  if (profile_enabled()) profile_end(st);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// Launch of the resident-operand weight gradient.  A unit is (expert, 256 columns, one of `split`
// ranges of p-blocks); `split` is chosen so that the last round of units over the resident
// clusters is as full as possible.
template <int EV>
static int launch_res(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int n_experts,
                      cudaStream_t st) {
  constexpr size_t smem = (size_t)kResTotalStages * kResStageBytes + 1024;
  auto kern = wgrad_resident_kernel<EV>;
  static PerDeviceInt max_clusters_of;
  const int dev = current_device();
  int max_clusters = (int)max_clusters_of.get(dev);
  if (max_clusters == 0) {
    MOLE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n;
    max_clusters_of.set(dev, n);
  }
  const int base = n_experts * (p.N / 256), pb = p.P / 256;
  int split = 1;
  double best = 0.0;
  for (int sp = 1; sp <= 8 && sp <= pb; sp *= 2) {
    const int units = base * sp;
    const int rounds = (units + max_clusters - 1) / max_clusters;
    const double fill = (double)units / ((double)rounds * max_clusters);
    if (fill > best + 0.02) { best = fill; split = sp; }
  }
  const int units = base * split;
  int clusters = max_clusters < units ? max_clusters : units;
  if (clusters <= 0) return MOLE_OK;
  if (profile_enabled()) profile_begin(st, p.epi);
  kern<<<2 * clusters, kThreads, smem, st>>>(ma, mb, p, split);
  if (profile_enabled()) profile_end(st);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

static void fill_sched(TcParams& p, const Schedule& s) {
  p.n_tiles = s.n_tiles;
  p.expert_tile_start = s.expert_tile_start;
  p.tile_row0 = s.tile_row0;
  p.tile_expert = s.tile_expert;
  p.tile_rows = s.tile_rows;
  p.expert_pair_start = s.expert_pair_start;
}

static bool takes_panel(const RowGemmArgs& a) {
  return a.panel && a.N % 256 == 0 && a.rowmap == nullptr && a.peers.n == 0 && a.c_y == nullptr &&
         a.max_rows_per_expert <= 8192;
}
// FC1 / dX2: a panel of 512 columns fills the TMEM, so its epilogue (activation, two stores per
// element: as long as the item's MMAs when the reduction is short) overlaps nothing.  Panels of
// at most 256 rows leave room for the next item's accumulator (measured: -5 % at K = 2048 and
// ~512 rows per expert, -5 to -8 % at K = 1024).
static int panel_split_of(const RowGemmArgs& a) { return a.epi == EPI_FC1 || a.epi == EPI_DACT; }
static int colsum_panels_of(int max_rows_per_expert) { return (max_rows_per_expert + 255) / 256; }

// The CTA-pair tile kernel sums too (per row tile), where it runs the dX2 launch: that is the
// many-rows-per-expert regime, in which its epilogue is hidden behind the main loop.
static bool tile_colsum(const RowGemmArgs& a) {
  return a.epi == EPI_DACT && a.colsum_ws != nullptr && !takes_panel(a) && a.N % 256 == 0 &&
         !a.single_cta && a.rowmap == nullptr;
}
bool tc_panel_colsum(const RowGemmArgs& a) {
  return a.epi == EPI_DACT && a.colsum_ws != nullptr && (takes_panel(a) || tile_colsum(a));
}
// room for either layout: [expert][panel][4][N] or [row tile][4][N]
int64_t tc_panel_colsum_bytes(int n_experts, int max_rows_per_expert, int N) {
  const int64_t per_expert = (max_rows_per_expert + kTileRows - 1) / kTileRows;     // >= its panels
  return (int64_t)n_experts * per_expert * 4 * N * (int64_t)sizeof(float);
}
int tc_panel_colsum_reduce(const RowGemmArgs& a, const SlotMap& gslot, int accumulate, void* out,
                           cudaStream_t st) {
  MOLE_REQUIRE(tc_panel_colsum(a), "no fused column sums for this launch");
  if (a.n_experts <= 0) return MOLE_OK;
  PanelColsumArgs r{};
  r.ws = a.colsum_ws;
  r.expert_tile_start = a.sched.expert_tile_start;
  r.tile_rows = a.sched.tile_rows;
  r.expert_pair_start = a.sched.expert_pair_start;
  r.tile_row0 = a.sched.tile_row0;
  r.tiles = tile_colsum(a) ? 1 : 0;
  r.N = a.N;
  r.panels = colsum_panels_of(a.max_rows_per_expert);
  r.split = panel_split_of(a);
  r.accumulate = accumulate;
  r.e_begin = a.e_begin;
  r.out = static_cast<__nv_bfloat16*>(out);
  r.gslot = gslot;
  dim3 grid((a.N + 255) / 256, a.n_experts);
  panel_colsum_reduce_kernel<<<grid, 256, 0, st>>>(r);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

int tc_row_gemm(const RowGemmArgs& a, cudaStream_t st) {
  MOLE_REQUIRE(a.N % 128 == 0 && a.K % kBK == 0, "tensor-core GEMM needs N %% 128 == 0 and K %% 64 == 0 (N=%d K=%d)", a.N, a.K);
  MOLE_REQUIRE(a.total_rows % kTileRows == 0, "row buffers must hold whole 128-row tiles");
  const int BN = a.N % 256 == 0 ? 256 : 128;
  const bool panel = takes_panel(a);
  const bool pair = BN == 256 && (!a.single_cta || panel);
  CUtensorMap ma, mb;
  PanelMaps pm;
  if (panel) {
    for (int i = 0; i < 4; ++i) {
      const uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.total_rows};
      const uint32_t box[2] = {kBK, (uint32_t)(64 >> i)};
      if (int rc = make_map(&pm.x[i], a.A, 2, dims, box)) return rc;
    }
  } else {
    const uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.total_rows};
    const uint32_t box[2] = {kBK, kBM};
    if (int rc = make_map(&ma, a.A, 2, dims, box)) return rc;
  }
  {
    // the weights are [n_slots][F][M] with M contiguous; as [N][K] that is N = F, K = M, as
    // [K][N] it is K = F, N = M: either way dims = {M, F, n_slots}
    const uint64_t inner = a.w_nk ? (uint64_t)a.K : (uint64_t)a.N;
    const uint64_t outer = a.w_nk ? (uint64_t)a.N : (uint64_t)a.K;
    MOLE_REQUIRE((int64_t)(inner * outer) == a.w_expert_stride, "weight stride mismatch");
    const uint64_t dims[3] = {inner, outer, (uint64_t)a.n_slots};
    const uint32_t box_k[3] = {kBK, (uint32_t)(pair ? 128 : BN), 1};   // a pair loads half each
    const uint32_t box_n[3] = {64, kBK, 1};
    if (int rc = make_map(&mb, a.W, 3, dims, a.w_nk ? box_k : box_n)) return rc;
  }
  TcParams p{};
  fill_sched(p, a.sched);
  p.n_experts = a.n_experts;
  p.e_begin = a.e_begin;
  p.N = a.N;
  p.K = a.K;
  p.P = 0;
  p.epi = a.epi;
  p.act = a.act;
  p.gelu_bwd = a.gelu_bwd;
  p.accumulate = 0;
  p.panel_split = panel_split_of(a);
  p.colsum_ws = tc_panel_colsum(a) ? a.colsum_ws : nullptr;
  p.colsum_panels = colsum_panels_of(a.max_rows_per_expert);
  p.colsum_tiles = tile_colsum(a) ? 1 : 0;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.aux = static_cast<const __nv_bfloat16*>(a.aux);
  p.out0 = static_cast<__nv_bfloat16*>(a.out0);
  p.out1 = static_cast<__nv_bfloat16*>(a.out1);
  p.fault = device_fault_word();
  p.slot = a.wslot;
  p.rowmap = a.rowmap;
  p.peer_n = a.peers.n;
  p.peer_rank = a.peers.rank;
  p.peer_L = a.peers.L;
  p.peer_Cs = a.peer_Cs;
  for (int q = 0; q < kMaxPeers; ++q) p.peer_base[q] = a.peers.base[q];
  p.c_perm = a.c_perm; p.c_offsets = a.c_offsets; p.c_counts = a.c_counts; p.c_gates = a.c_gates;
  p.c_y = static_cast<__nv_bfloat16*>(a.c_y); p.c_k = a.c_k; p.c_Cs = a.c_Cs;
  MOLE_REQUIRE(a.peers.n == 0 || a.rowmap != nullptr, "peer scatter needs the row map");
  MOLE_REQUIRE(a.rowmap == nullptr || a.epi == EPI_BIAS || a.epi == EPI_STORE,
               "only FC2 / dX outputs can be scattered");
  const int max_items = a.sched.max_tiles * (a.N / BN);
  for (const void* q : {a.bias, a.aux, (const void*)a.out0, (const void*)a.out1})
    MOLE_REQUIRE((reinterpret_cast<uintptr_t>(q) & 31) == 0, "epilogue operand %p not 32-byte aligned", q);
  MOLE_REQUIRE(a.c_y == nullptr || (!pair && a.rowmap == nullptr && (a.epi == EPI_BIAS || a.epi == EPI_STORE)),
               "the fused combine needs the one-CTA kernel and rows that are not scattered");
  if (panel) pm.w = mb;
  // one kernel per (operand layout, tile shape, epilogue variant)
#define MOLE_ROWS(KM, EV)                                                                    \
  return panel ? launch_panel<KM, EV>(pm, p, max_items, a.max_rows_per_expert, st)                               \
         : pair ? launch_tc2<TC_ROWS, KM, EV>(ma, mb, p, max_items, st)                      \
              : BN == 256 ? launch_tc<TC_ROWS, KM, 256, EV>(ma, mb, p, max_items, st)        \
                          : launch_tc<TC_ROWS, KM, 128, EV>(ma, mb, p, max_items, st)
  const bool relu = a.act == MOLE_ACT_RELU;
  if (a.epi == EPI_FC1) {
    MOLE_REQUIRE(a.w_nk, "FC1 reads its weights K-major");
    if (a.bias) { if (relu) { MOLE_ROWS(true, EV_FC1_RELU_B); } else { MOLE_ROWS(true, EV_FC1_GELU_B); } }
    if (relu) { MOLE_ROWS(true, EV_FC1_RELU); } else { MOLE_ROWS(true, EV_FC1_GELU); }
  }
  if (a.epi == EPI_DACT) {
    MOLE_REQUIRE(a.w_nk, "dX2 reads its weights K-major");
    if (relu) { MOLE_ROWS(true, EV_DACT_RELU); }
    if (a.gelu_bwd == MOLE_GELU_BWD_TANH) { MOLE_ROWS(true, EV_DACT_TANH); }
    MOLE_ROWS(true, EV_DACT_GELU);
  }
  MOLE_REQUIRE(!a.w_nk, "FC2 / dX read their weights N-major");
  if (a.epi == EPI_BIAS && a.bias) { MOLE_ROWS(false, EV_BIAS); }
  MOLE_ROWS(false, EV_STORE);
#undef MOLE_ROWS
}

int tc_wgrad(const WgradArgs& a, cudaStream_t st) {
  MOLE_REQUIRE(a.P % kBM == 0 && a.Q % 128 == 0, "tensor-core wgrad needs F %% 128 == 0 and M %% 128 == 0");
  MOLE_REQUIRE(a.total_rows % kTileRows == 0, "row buffers must hold whole 128-row tiles");
  if (a.n_experts <= 0) return MOLE_OK;
  const int BN = a.Q % 256 == 0 ? 256 : 128;
  CUtensorMap ma, mb;
  const uint32_t box[2] = {64, kWBK};
  {
    const uint64_t dims[2] = {(uint64_t)a.P, (uint64_t)a.total_rows};
    if (int rc = make_map(&ma, a.A, 2, dims, box)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a.Q, (uint64_t)a.total_rows};
    if (int rc = make_map(&mb, a.B, 2, dims, box)) return rc;
  }
  TcParams p{};
  fill_sched(p, a.sched);
  p.n_experts = a.n_experts;
  p.e_begin = a.e_begin;
  p.N = a.Q;
  p.K = 0;
  p.P = a.P;
  p.epi = EPI_WGRAD;
  p.accumulate = a.accumulate;
  p.out0 = static_cast<__nv_bfloat16*>(a.out);
  p.fault = device_fault_word();
  p.slot = a.gslot;
  MOLE_REQUIRE((reinterpret_cast<uintptr_t>(a.out) & 31) == 0, "gradient base not 32-byte aligned");
  const int max_items = a.n_experts * (a.P / kBM) * (a.Q / BN);
  // an expert's 64-row stages: at most two per 128-row tile
  const int max_stages = 2 * a.max_tiles_per_expert;
  if (a.resident && BN == 256 && a.P % 256 == 0 && max_stages > 0 && max_stages <= kResMaxResident) {
    if (a.accumulate) return launch_res<EV_WGRAD_ACC>(ma, mb, p, a.n_experts, st);
    return launch_res<EV_WGRAD>(ma, mb, p, a.n_experts, st);
  }
#define MOLE_WG(EV)                                                                               \
  if (BN == 256 && a.P % 256 == 0 && !a.single_cta)                                               \
    return launch_tc2<TC_WGRAD, true, EV>(ma, mb, p, a.n_experts * (a.P / 256) * (a.Q / 256), st); \
  return BN == 256 ? launch_tc<TC_WGRAD, true, 256, EV>(ma, mb, p, max_items, st)                 \
                   : launch_tc<TC_WGRAD, true, 128, EV>(ma, mb, p, max_items, st)
  if (a.accumulate) { MOLE_WG(EV_WGRAD_ACC); }
  MOLE_WG(EV_WGRAD);
#undef MOLE_WG
}

}  // namespace mole
