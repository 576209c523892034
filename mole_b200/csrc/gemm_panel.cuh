// Panel kernel: the rows-mode grouped GEMM with the operand roles swapped.  Included by
// gemm_tc.cu (it uses that file's PTX wrappers, TcParams and epilogue traits).
//
// The tile kernels put 128 rows of an expert on the M side of the MMA: an expert with 264 rows
// pays for 384, and every extra tile streams the expert's weights through shared memory again.
// The GEMMs run at the rate shared memory can be refilled (bytes in flight / load latency), so
// what counts is the work done per byte staged.  Here the WEIGHTS are the M operand -- a CTA pair
// (cta_group::2) takes 256 output features of one expert, 128 per SM, always full -- and the
// expert's rows are the N operand: D^T[feature][row] = W[feature][k] * X[row][k].  A work item is
// (expert, 256 features, panel of up to 512 rows): up to 256 rows go into one accumulator
// (N = rows rounded up to 16), more into two accumulators of equal size (N1 = N2, rows rounded up
// to 32) that are fed by alternating MMAs from the same staged weights.  264 rows cost 288, and
// the weights cross shared memory once per expert.
//
// TMEM holds 512 columns.  Items alternate between the two ends of it ([0, c) and [512 - c, 512));
// while the two regions do not overlap, the epilogue of one item runs under the main loop of
// the next; where they do (c + c' > 512) the issuer first waits for the previous item's drain.
//
// The accumulator comes out transposed: a thread of the epilogue owns one feature and reads 16
// rows of it per tcgen05.ld; bias is one scalar per thread.  FC2 / dX store it as it comes (a
// warp's store instruction writes 32 neighbouring features of one row, 64 contiguous bytes);
// FC1 / dX2 turn each 16 x 32 block round in shared memory first and use 16-byte accesses (see
// "FC1 / dX2 epilogue" below).  Experts of more than 320 rows are cut into panels of at most 256
// rows for FC1 / dX2 (TcParams::panel_split), so that the next item's accumulator fits beside.
//
// Needs every expert's rows in one contiguous run (one source rank, or the compacted layout)
// and outputs that stay in place (no row map).
#pragma once

constexpr uint32_t kPanelABytes = 128 * kBK * 2;      // 128 features x 64 K per CTA and stage

struct PanelMaps {
  CUtensorMap w;        // weights: box 64 K x 128 features (K-major) or 64 features x 64 K (N-major)
  CUtensorMap x[4];     // rows [total_rows][K]: boxes of 64 K x {64, 32, 16, 8} rows
};

struct PanelItem {
  int valid;
  int el;          // expert relative to e_begin
  int n0;          // first of the pair's 256 output features
  int row0;        // first row of the panel
  int n1, n2;      // columns of the two accumulators (multiples of 16; n2 may be 0; n1 = 0: nothing to do)
  int pan;         // which of the expert's panels
};

// Panels of an expert with `pairs` = ceil(tiles / 2) pairs of row tiles: ceil(rows / 512), or, with
// `split`, one per 256 rows once the expert has more than 320 rows.
__device__ __forceinline__ int panel_count(int rows, int pairs, int split) {
  return (split && rows > 320) ? pairs : (pairs + 1) >> 1;
}

// Experts are visited in the order of falling row counts (`order`, built once per CTA): items of
// more than 256 rows cost about 1.3 of the others, and a launch may have only half a dozen items
// per cluster, so the round-robin assignment must deal both kinds out evenly.
// `istart` = prefix over the ORDERED experts of their panels, ceil(rows / 512); `start` =
// expert_tile_start (by expert).
__device__ __forceinline__ PanelItem decode_panel(const TcParams& p, const int* start, const int* istart,
                                                  const uint8_t* order, int item) {
  PanelItem w;
  w.valid = 0;
  const int nb = p.N / 256;
  if (item < 0 || item >= istart[p.n_experts] * nb) return w;
  int lo = 0, hi = p.n_experts;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (istart[mid] * nb <= item) lo = mid; else hi = mid;
  }
  const int ps = istart[lo], np = istart[lo + 1] - ps;
  const int local = item - ps * nb;
  const int pan = local % np;            // panels of a feature block are neighbours: they share W through L2
  const int e = order[lo];
  const int ts = start[e], te = start[e + 1];
  const int rows = (te - ts - 1) * kTileRows + p.tile_rows[te - 1];
  const int per = (((rows + np - 1) / np) + 31) & ~31;      // <= 512
  const int left = rows - pan * per;
  w.valid = 1;
  w.el = e;
  w.n0 = (local / np) * 256;
  w.row0 = p.tile_row0[ts] + pan * per;
  w.n1 = w.n2 = 0;
  w.pan = pan;
  if (left > 0) {
    const int r = min(per, left);
    if (r <= 256) w.n1 = (r + 15) & ~15;
    else w.n1 = w.n2 = ((r + 31) & ~31) >> 1;
  }
  return w;
}
// Columns of an item without reading its rows' position: what the epilogue needs of the NEXT item
__device__ __forceinline__ int panel_cols(const PanelItem& w) { return w.valid ? w.n1 + w.n2 : 0; }

__device__ __forceinline__ uint16_t bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void st_b16(__nv_bfloat16* p, uint16_t v) {
  asm volatile("st.global.b16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
}
// One lane polls, the warp gets the answer (or every lane polls: `one` = false).
__device__ __forceinline__ bool warp_wait(bool one, uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* fault, int code) {
  if (!one) return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, fault, code));
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, fault, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// The epilogue of 16 rows x one feature per thread for FC2 / dX (bias or plain store)
template <int EV>
__device__ __forceinline__ void panel_store16(const TcParams& p, const uint32_t (&r)[16], int64_t off,
                                              float bias) {
#pragma unroll
  for (int i = 0; i < 16; ++i)
    st_b16(p.out0 + off + (int64_t)i * p.N, bf16_bits(__uint_as_float(r[i]) + bias));
}

// ---- FC1 / dX2 epilogue of the panel kernel -----------------------------------------------
// These two epilogues are bound by instruction issue (activation, rounding, two outputs), so
// they are written for few instructions per element:
//   * the arithmetic runs on pairs of rows with the packed fp32 instructions (fma / mul / add
//     .f32x2), in the same order of operations as the scalar code: results are bit-identical;
//   * the transposed accumulator (thread = feature, registers = rows) is turned round in a 1 KB
//     shared-memory strip per warp, so that global memory sees 16-byte accesses: a lane stores
//     (or, for the pre-activations of dX2, loads) eight neighbouring features of two rows, where
//     it would otherwise issue sixteen 2-byte accesses with sixteen addresses.
// Strip layout: word (rp, l) = rows (2 rp, 2 rp + 1) of feature l, at rp * 32 + (l ^ 4 (rp & 1));
// the swap of neighbouring groups of four lanes in odd row pairs keeps the 16-byte accesses of
// the row side free of bank conflicts.
struct PanelStrip {
  uint32_t* we;        // feature side: this lane's word of an even / odd row pair (+ 32 per pair)
  uint32_t* wo;
  uint4* ra;           // row side: features 0-3 / 4-7 of this lane's (row pair, group of eight)
  uint4* rb;
  __device__ __forceinline__ void init(uint32_t* strip, int lane) {
    we = strip + lane;
    wo = strip + (lane ^ 4);
    const int rp = lane >> 2, g = lane & 3;
    uint4* s4 = reinterpret_cast<uint4*>(strip);
    ra = s4 + rp * 8 + 2 * g + (rp & 1);
    rb = s4 + rp * 8 + 2 * g + 1 - (rp & 1);
  }
  __device__ __forceinline__ void put(const uint32_t (&w)[8]) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) ((i & 1) ? wo : we)[32 * i] = w[i];
  }
  __device__ __forceinline__ void get(uint32_t (&w)[8]) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = ((i & 1) ? wo : we)[32 * i];
  }
  // eight features of the lane's two rows, as they lie in memory
  __device__ __forceinline__ void take_rows(uint4& a, uint4& b) const {
    const uint4 lo = *ra, hi = *rb;
    a = make_uint4(__byte_perm(lo.x, lo.y, 0x5410), __byte_perm(lo.z, lo.w, 0x5410),
                   __byte_perm(hi.x, hi.y, 0x5410), __byte_perm(hi.z, hi.w, 0x5410));
    b = make_uint4(__byte_perm(lo.x, lo.y, 0x7632), __byte_perm(lo.z, lo.w, 0x7632),
                   __byte_perm(hi.x, hi.y, 0x7632), __byte_perm(hi.z, hi.w, 0x7632));
  }
  __device__ __forceinline__ void put_rows(const uint4& a, const uint4& b) const {
    *ra = make_uint4(__byte_perm(a.x, b.x, 0x5410), __byte_perm(a.x, b.x, 0x7632),
                     __byte_perm(a.y, b.y, 0x5410), __byte_perm(a.y, b.y, 0x7632));
    *rb = make_uint4(__byte_perm(a.z, b.z, 0x5410), __byte_perm(a.z, b.z, 0x7632),
                     __byte_perm(a.w, b.w, 0x5410), __byte_perm(a.w, b.w, 0x7632));
  }
};
__device__ __forceinline__ void st_v4(__nv_bfloat16* p, const uint4& v) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_v4(const __nv_bfloat16* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
constexpr bool panel_heavy(int epi) { return epi == EPI_FC1 || epi == EPI_DACT; }
constexpr int kPanelStripWords = 256;      // 1 KB per epilogue warp (FC1 / dX2 only)

// `stages` x `stage_bytes` of dynamic shared memory: a stage is this CTA's 128 features x 64 K of
// weights (16 KB) followed by its share of the panel's rows (up to `stage_bytes` - 16 KB).
constexpr int kPanelMaxStages = 8;
template <bool W_KMAJOR, int EV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
panel_gemm_kernel(const __grid_constant__ PanelMaps maps, const __grid_constant__ TcParams p,
                  const int stages, const uint32_t stage_bytes) {
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kBoxBytes = 128 * kBK;             // one 64-feature box of N-major weights
  // f32 accumulate, bf16 operands, A (weights) K-major or MN-major, B (rows) K-major, M = 256
  constexpr uint32_t kIdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((W_KMAJOR ? 0u : 1u) << 15) |
                                  ((uint32_t)(256 >> 4) << 24);
  using Ev = EvTraits<EV>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t bars[2 * kPanelMaxStages + 7];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag_s;
  __shared__ int start_s[kMaxLocalExperts + 1], istart_s[kMaxLocalExperts + 1];    // see decode_item
  __shared__ int pairs_s[kMaxLocalExperts + 1], rows_s[kMaxLocalExperts];
  __shared__ uint8_t order_s[kMaxLocalExperts];
  __shared__ __align__(16) uint32_t xstrip_s[panel_heavy(Ev::epi) ? kEpiWarps * kPanelStripWords : 4];
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kPanelMaxStages]);
  const uint32_t tfull0 = smem_u32(&bars[2 * kPanelMaxStages]), tempty0 = smem_u32(&bars[2 * kPanelMaxStages + 2]);
  const uint32_t drain0 = smem_u32(&bars[2 * kPanelMaxStages + 4]);      // used only after an abort
  const uint32_t tovl0 = smem_u32(&bars[2 * kPanelMaxStages + 5]);       // overlap columns drained
  const uint32_t smem_base = smem_u32(smem);
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int nkb = p.K / kBK;

  for (int i = threadIdx.x; i <= p.n_experts; i += kThreads) {
    start_s[i] = p.expert_tile_start[i];
    pairs_s[i] = p.expert_pair_start[i];
  }
  __syncthreads();
  // rank of every expert by falling number of tile pairs (ties: by index): its place in the order
  for (int e = threadIdx.x; e < p.n_experts; e += kThreads) {
    const int ts = start_s[e], te = start_s[e + 1];
    rows_s[e] = te > ts ? (te - ts - 1) * kTileRows + p.tile_rows[te - 1] : 0;
    const int mine = pairs_s[e + 1] - pairs_s[e];
    int rk = 0;
    for (int o = 0; o < p.n_experts; ++o) {
      const int other = pairs_s[o + 1] - pairs_s[o];
      rk += (other > mine) || (other == mine && o < e);
    }
    order_s[rk] = (uint8_t)e;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    mbar_init(drain0, 1);
    for (int s = 0; s < kPanelMaxStages; ++s) {
      mbar_init(full0 + 8 * s, 1);               // the even CTA's arrive.expect_tx
      mbar_init(empty0 + 8 * s, 1);              // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 2 * kEpiWarps); // epilogue warps of both CTAs
      mbar_init(tovl0 + 8 * a, 2 * kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // panels per expert, in the order: ceil(pairs of tiles / 2) = ceil(rows / 512); with
    // `panel_split` an expert of more than 320 rows gets one panel per 256 rows instead
    int run = 0;
    for (int i = 0; i < p.n_experts; ++i) {
      const int e = order_s[i];
      const int pairs = pairs_s[e + 1] - pairs_s[e];
      istart_s[i] = run;
      run += panel_count(rows_s[e], pairs, p.panel_split);
    }
    istart_s[p.n_experts] = run;
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
    // ------------------------------- TMA producer (both CTAs, whole warp) --------------
    // A stage is one or two weight boxes and the CTA's share of the panel's rows -- half of each
    // accumulator's rows, cut into boxes of 64, 32, 16 and 8 rows; every box has its own lane.
    int stage = 0;
    uint32_t phase = 0, issued = 0;
    bool ok = true;
    for (int item = cluster_id; ok; item += n_clusters) {
      const PanelItem w = decode_panel(p, start_s, istart_s, order_s, item);
      if (!w.valid) break;
      if (w.n1 == 0) continue;
      const int slot = p.slot.s[p.e_begin + w.el];
      const int h1 = w.n1 >> 1, h2 = w.n2 >> 1;          // rows this CTA stages per accumulator
      const uint32_t tx = 2u * (kPanelABytes + (uint32_t)(h1 + h2) * 128u);
      const int f0 = w.n0 + 128 * (int)rank;           // this CTA's features
      // what this lane loads in every stage of the item: lanes 2..6 the first accumulator's rows,
      // lanes 7..11 the second's
      int kind = -1, off = 0, srow = 0;                // kind 0..3: a box of 64 >> kind rows
      {
        const int part = lane >= 7 ? 1 : 0;
        const int l = lane - (part ? 7 : 2);           // 0, 1: boxes of 64; 2, 3, 4: 32, 16, 8
        const int h = part ? h2 : h1;
        const int n64 = h >> 6, rem = h & 63;
        if (lane >= 2 && lane < 12) {
          if (l < 2) { if (l < n64) { kind = 0; off = 64 * l; } }
          else if (l == 2) { if (rem & 32) { kind = 1; off = 64 * n64; } }
          else if (l == 3) { if (rem & 16) { kind = 2; off = 64 * n64 + (rem & 32); } }
          else { if (rem & 8) { kind = 3; off = 64 * n64 + (rem & 48); } }
        }
        // accumulator 1 holds the panel's rows [0, n1), accumulator 2 rows [n1, n1 + n2); this CTA
        // supplies the lower (rank 0) or upper half of each
        srow = w.row0 + (part ? w.n1 + h2 * (int)rank : h1 * (int)rank) + off;
        off += part ? h1 : 0;                          // position in the stage's row area
      }
      for (int kb = 0; kb < nkb; ++kb) {
        ok = warp_wait(false, empty0 + 8 * stage, phase ^ 1, abort_flag, p.fault, 21);
        if (!ok) break;
        const uint32_t bar = (full0 + 8 * stage) & kPeerMask;     // the even CTA's barrier
        const uint32_t sa = smem_base + stage * stage_bytes, sb = sa + kPanelABytes;
        if (leader && lane == 0) mbar_expect_tx(full0 + 8 * stage, tx);
        if (W_KMAJOR) {
          if (lane == 0) tma2_load_3d(sa, &maps.w, bar, kb * kBK, f0, slot);
        } else {
          if (lane < 2) tma2_load_3d(sa + lane * kBoxBytes, &maps.w, bar, f0 + 64 * lane, kb * kBK, slot);
        }
        if (kind >= 0) tma2_load_2d(sb + off * 128, &maps.x[kind], bar, kb * kBK, srow);
        ++issued;
        if (++stage == stages) { stage = 0; phase ^= 1; }
      }
    }
    // both CTAs' loads complete on the even CTA's barriers: it waits for the pair
    if (leader && lane == 0 && *abort_flag) drain_loads(full0, stages, issued);
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA only) -----------------------
    if (lane == 0 && leader) {
      int stage = 0, acc = 0, c_prev = 0;
      uint32_t phase = 0, aph0 = 0, aph1 = 0;           // phase of each end's barriers
      bool ok = true;
      for (int item = cluster_id; ok; item += n_clusters) {
        const PanelItem w = decode_panel(p, start_s, istart_s, order_s, item);
        if (!w.valid) break;
        if (w.n1 == 0) continue;
        const int c = w.n1 + w.n2;
        if (!(ok = mbar_wait(tempty0 + 8 * acc, (acc ? aph1 : aph0) ^ 1, abort_flag, p.fault, 22))) break;
        // the previous item sits at the other end of TMEM: if the two overlap, wait until its
        // epilogue has drained the columns they share (it takes those first)
        if (c + c_prev > (int)kTmemCols &&
            !(ok = mbar_wait(tovl0 + 8 * (acc ^ 1), (acc ? aph0 : aph1) ^ 1, abort_flag, p.fault, 22))) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (acc ? kTmemCols - c : 0);
        const uint32_t idesc1 = kIdescBase | ((uint32_t)(w.n1 >> 3) << 17);
        const uint32_t idesc2 = kIdescBase | ((uint32_t)(w.n2 >> 3) << 17);
        const uint32_t b2off = (uint32_t)(w.n1 >> 1) * 128u;
        // the two forms of the K loop are separate straight-line code: a branch between the MMAs of
        // a stage slows their issue
        auto k_loop = [&](auto dual) {
          for (int kb = 0; kb < nkb; ++kb) {
            if (!(ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.fault, 23))) break;
            tcgen05_fence_after();
            const uint32_t sa = smem_base + stage * stage_bytes, sb = sa + kPanelABytes;
#pragma unroll
            for (int ks = 0; ks < kBK / kUmmaK; ++ks) {
              const uint64_t ad = W_KMAJOR ? make_desc(sa + ks * (kUmmaK * 2), 16, 1024)
                                           : make_desc(sa + ks * (kUmmaK * 128), kBoxBytes, 1024);
              tcgen05_mma2_bf16(d_tmem, ad, make_desc(sb + ks * (kUmmaK * 2), 16, 1024), idesc1,
                                (kb | ks) ? 1u : 0u);
              if (decltype(dual)::value)
                tcgen05_mma2_bf16(d_tmem + w.n1, ad, make_desc(sb + b2off + ks * (kUmmaK * 2), 16, 1024),
                                  idesc2, (kb | ks) ? 1u : 0u);
            }
            tcgen05_commit2(empty0 + 8 * stage);
            if (++stage == stages) { stage = 0; phase ^= 1; }
          }
        };
        if (w.n2) k_loop(std::true_type{}); else k_loop(std::false_type{});
        if (!ok) break;
        tcgen05_commit2(tfull0 + 8 * acc);
        if (acc) aph1 ^= 1; else aph0 ^= 1;
        acc ^= 1;
        c_prev = c;
      }
      if (*abort_flag) {                      // MMAs already issued retire before the TMEM goes
        tcgen05_commit2(drain0);
        mbar_drain(drain0, 0, globaltimer_ns() + 200000000ull);
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -----------------------------
    // warp -> 32 features (the TMEM lanes it may read) and every fourth chunk of 16 rows
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;
    int acc = 0;
    uint32_t aph0 = 0, aph1 = 0;                      // phase of each end's barriers
    for (int item = cluster_id;; item += n_clusters) {
      const PanelItem w = decode_panel(p, start_s, istart_s, order_s, item);
      if (!w.valid) break;
      const int f = w.n0 + 128 * (int)rank + 32 * quarter + lane;
      // dX2 with fused column sums: this warp's part of sum_rows dX1[:, f] for the panel
      float* cs_out = nullptr;
      if (Ev::epi == EPI_DACT && p.colsum_ws != nullptr)
        cs_out = p.colsum_ws + ((int64_t)(w.el * p.colsum_panels + w.pan) * 4 + grp) * p.N + f;
      if (w.n1 == 0) {
        if (cs_out) *cs_out = 0.f;
        continue;
      }
      const int c = w.n1 + w.n2;
      const int slot = p.slot.s[p.e_begin + w.el];
      const int64_t obase = (int64_t)w.row0 * p.N + f;         // element (row0, f) of the outputs
      float bias = 0.f;
      if (Ev::bias) bias = __bfloat162float(p.bias[(int64_t)slot * p.N + f]);
      // Columns [ov_lo, ov_hi) of this item (local numbering) are where the next item's
      // accumulators will sit: they are drained first and released on their own barrier.
      int ov_lo = 0, ov_hi = 0;
      {
        const int c_next = panel_cols(decode_panel(p, start_s, istart_s, order_s, item + n_clusters));
        if (c + c_next > (int)kTmemCols) {
          if (acc) { ov_lo = 0; ov_hi = c + c_next - (int)kTmemCols; }
          else { ov_lo = (int)kTmemCols - c_next; ov_hi = c; }
        }
      }
      // This warp's chunks of 16 rows in drain order: those inside the shared columns first.
      int it_pass = 0, it_c = grp * 16 - 64;
      auto next_chunk = [&]() -> int {
        while (it_pass < 2) {
          it_c += 64;
          if (it_c >= c) { ++it_pass; it_c = grp * 16 - 64; continue; }
          const bool inside = it_c >= ov_lo && it_c < ov_hi;
          if (inside == (it_pass == 0)) return it_c;
        }
        return -1;
      };
      int cur = next_chunk(), cur_pass = it_pass;
      const uint32_t taddr0 = ((uint32_t)(quarter * 32) << 16) + (acc ? kTmemCols - c : 0);
      auto release_shared = [&]() {                     // the shared columns are free
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster((tovl0 + 8 * acc) & kPeerMask);
      };
      if (panel_heavy(Ev::epi)) {
        PanelStrip xs;
        xs.init(xstrip_s + (warp - 2) * kPanelStripWords, lane);
        // row side: this lane's two rows (2 rp, 2 rp + 1 of a chunk) and eight features
        const int64_t rbase = ((int64_t)w.row0 + 2 * (lane >> 2)) * p.N + (f - lane) + 8 * (lane & 3);
        // dX2: the pre-activations of a chunk are fetched one chunk ahead, those of the first
        // chunk before the wait for the accumulator
        uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
        if (Ev::epi == EPI_DACT && cur >= 0) {
          const __nv_bfloat16* src = p.aux + rbase + (int64_t)cur * p.N;
          xa = ld_v4(src);
          xb = ld_v4(src + p.N);
        }
        if (!warp_wait(false, tfull0 + 8 * acc, acc ? aph1 : aph0, abort_flag, p.fault, 24))
          break;                                        // nothing is stored for this item
        tcgen05_fence_after();
        bool released = false;
        if (cur < 0 || cur_pass == 1) { release_shared(); released = true; }
        const uint64_t bias2 = f2_dup(bias);
        float csum = 0.f;
        while (cur >= 0) {
          const int nxt = next_chunk(), nxt_pass = it_pass;
          const int64_t o = rbase + (int64_t)cur * p.N;
          uint32_t xw[8], ow[8];
          if (Ev::epi == EPI_DACT) {
            __syncwarp();
            xs.put_rows(xa, xb);
            __syncwarp();
            xs.get(xw);
            if (nxt >= 0) {
              const __nv_bfloat16* src = p.aux + rbase + (int64_t)nxt * p.N;
              xa = ld_v4(src);
              xb = ld_v4(src + p.N);
            }
          }
          uint32_t r[16];
          tmem_ld16(tmem_base + taddr0 + cur, r);
          tmem_ld_wait();
          uint4 ra, rb;
          if (Ev::epi == EPI_FC1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
              if (Ev::bias) f2_unpack(f2_add(f2_pack(s0, s1), bias2), s0, s1);
              xw[i] = pack_bf16(s0, s1);
              // the activation is taken of the rounded pre-activation, as backward sees it
              ow[i] = act_fwd_pair<Ev::act>(xw[i]);
            }
            __syncwarp();
            xs.put(xw);
            __syncwarp();
            xs.take_rows(ra, rb);
            st_v4(p.out0 + o, ra);
            st_v4(p.out0 + o + p.N, rb);
            __syncwarp();
            xs.put(ow);
            __syncwarp();
            xs.take_rows(ra, rb);
            st_v4(p.out1 + o, ra);
            st_v4(p.out1 + o + p.N, rb);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              ow[i] = act_bwd_pair<Ev::act, Ev::gbwd>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), xw[i]);
              csum += bf16_lo(ow[i]) + bf16_hi(ow[i]);       // of the stored (rounded) values
            }
            __syncwarp();
            xs.put(ow);
            __syncwarp();
            xs.take_rows(ra, rb);
            st_v4(p.out0 + o, ra);
            st_v4(p.out0 + o + p.N, rb);
          }
          if (!released && cur_pass == 0 && (nxt < 0 || nxt_pass == 1)) { release_shared(); released = true; }
          cur = nxt;
          cur_pass = nxt_pass;
        }
        if (cs_out) *cs_out = csum;
      } else {
        if (!warp_wait(false, tfull0 + 8 * acc, acc ? aph1 : aph0, abort_flag, p.fault, 24))
          break;                                        // nothing is stored for this item
        tcgen05_fence_after();
        bool released = false;
        if (cur < 0 || cur_pass == 1) { release_shared(); released = true; }
        while (cur >= 0) {
          const int nxt = next_chunk(), nxt_pass = it_pass;
          uint32_t r[16];
          tmem_ld16(tmem_base + taddr0 + cur, r);
          tmem_ld_wait();
          panel_store16<EV>(p, r, obase + (int64_t)cur * p.N, bias);
          if (!released && cur_pass == 0 && (nxt < 0 || nxt_pass == 1)) { release_shared(); released = true; }
          cur = nxt;
          cur_pass = nxt_pass;
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster((tempty0 + 8 * acc) & kPeerMask);
      if (acc) aph1 ^= 1; else aph0 ^= 1;
      acc ^= 1;
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

// Column sums that a dX2 launch left as partial sums -- the panel kernel per (expert, panel, one of
// the four row groups of the epilogue, feature), the CTA-pair tile kernel per (row tile, one of
// the tile's four 32-row quarters, feature) -- added in a fixed order: bit-reproducible.
struct PanelColsumArgs {
  const float* ws;
  const int32_t* expert_tile_start;
  const int32_t* tile_rows;
  const int32_t* expert_pair_start;
  const int32_t* tile_row0;    // tile layout (the CTA-pair tile kernel's partials, [row0 / 128][4][N])
  int tiles;                   // 1: tile layout
  int N, panels, split, accumulate, e_begin;
  __nv_bfloat16* out;          // [n_slots, N]
  SlotMap gslot;
};
__global__ void __launch_bounds__(256)
panel_colsum_reduce_kernel(const __grid_constant__ PanelColsumArgs a) {
  const int el = blockIdx.y;
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n >= a.N) return;
  const int ts = a.expert_tile_start[el], te = a.expert_tile_start[el + 1];
  const int rows = te > ts ? (te - ts - 1) * kTileRows + a.tile_rows[te - 1] : 0;
  float v = 0.f;
  if (a.tiles) {
    for (int t = ts; t < te; ++t) {
      const float* part = a.ws + (int64_t)(a.tile_row0[t] / kTileRows) * 4 * a.N + n;
      for (int q = 0; q < 4; ++q) v += part[(int64_t)q * a.N];
    }
  } else {
    const int np = panel_count(rows, a.expert_pair_start[el + 1] - a.expert_pair_start[el], a.split);
    for (int i = 0; i < np * 4; ++i) v += a.ws[((int64_t)el * a.panels * 4 + i) * a.N + n];
  }
  __nv_bfloat16* out = a.out + (int64_t)a.gslot.s[a.e_begin + el] * a.N + n;
  if (a.accumulate) v += __bfloat162float(*out);
  *out = __float2bfloat16_rn(v);
}

// =========================================================================================
// Weight gradient with one operand resident in shared memory.
//
// gW_e[p, q] = sum_r A[r, p] * B[r, q] over the rows r of expert e: the reduction is short (an
// expert's few hundred rows) and the output large ([F, M] per expert), so the tile kernels load
// (128 + 256) x rows operand elements for every 128 x 256 outputs -- three times the bytes they
// write -- and run at the rate shared memory can be filled through L2, not at the rate HBM takes
// the gradient.  Here a CTA pair takes (expert, 256 columns q) and keeps B[:, q-block] -- all
// rows of the expert, 128 columns per CTA -- in shared memory while it walks down the expert's
// p-blocks of 256, streaming only A: operand bytes per output tile drop from 240 KB to ~85 KB.
//
//   shared memory per CTA: twelve stages of 64 rows x 128 columns (16 KB each).  A unit's resident
//   operand takes as many as the expert has 64-row stages (at most eight; the host checks the
//   bound and falls back to the tile kernel beyond it), the ring of the streamed operand the
//   rest: the loads in flight, which set the kernel's pace, get every byte that is left.
//   (Measured: letting stages beyond the eighth follow A through the ring, or keeping fewer than
//   eight resident, brings an expert of ~512 rows to the tile kernel's time, not below it.)
//
// Barriers as in tc2_gemm_kernel, plus bfull (resident operand landed; armed by the even CTA,
// completed by both CTAs' loads) and bfree (every MMA that reads the resident operand has
// retired; a multicast commit).
constexpr int kResTotalStages = 12;
constexpr int kResMaxResident = 8;
constexpr uint32_t kResStageBytes = 128 * kWBK * 2;      // 16 KB: 64 rows x 128 columns, two boxes

struct ResUnit {
  int valid;
  int el;
  int q0;            // first of the pair's 256 output columns
  int pb0, pb1;      // p-blocks (of 256 rows of the output) this unit walks
  int row0, rows;    // the expert's rows: one contiguous run (0 rows: the gradient is zero)
};
// Stage s of an expert covers rows [row0 + 64 s, ...): its number of 16-row MMA steps
__device__ __forceinline__ int res_ksteps(int rows, int s) {
  const int left = rows - s * kWBK;
  return left >= kWBK ? kWBK / kUmmaK : (left + kUmmaK - 1) / kUmmaK;
}

__device__ __forceinline__ ResUnit decode_res(const TcParams& p, int unit, int split) {
  ResUnit w;
  w.valid = 0;
  const int qb = p.N / 256, pb = p.P / 256;
  if (unit >= p.n_experts * qb * split) return w;
  w.valid = 1;
  w.el = unit / (qb * split);
  const int r = unit - w.el * qb * split;
  // the q-blocks of one range of p are neighbours: they stream the same A through L2
  w.q0 = (r % qb) * 256;
  const int sp = r / qb;
  w.pb0 = (int)((int64_t)pb * sp / split);
  w.pb1 = (int)((int64_t)pb * (sp + 1) / split);
  const int t0 = p.expert_tile_start[w.el], t1 = p.expert_tile_start[w.el + 1];
  w.rows = t1 > t0 ? (t1 - t0 - 1) * kTileRows + p.tile_rows[t1 - 1] : 0;
  w.row0 = t1 > t0 ? p.tile_row0[t0] : 0;
  return w;
}

template <int EV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
wgrad_resident_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ TcParams p, const int split) {
  constexpr int STAGES = kResTotalStages;       // barriers; a unit's ring has 12 - (its resident stages)
  constexpr int RES = kResMaxResident;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kBoxBytes = 128 * kWBK;            // one box: 64 columns x 64 rows
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                              ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 7];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag_s;
  __shared__ __align__(16) uint8_t store_strip[kEpiWarps][kStripBytes];
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
  const uint32_t drain0 = smem_u32(&bars[2 * STAGES + 4]);      // used only after an abort
  const uint32_t bfull = smem_u32(&bars[2 * STAGES + 5]), bfree = smem_u32(&bars[2 * STAGES + 6]);
  const uint32_t res_base = smem_u32(smem);      // a unit's resident stages, followed by its ring
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    mbar_init(drain0, 1);
    mbar_init(bfull, 1);
    mbar_init(bfree, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 2 * kEpiWarps);
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
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs, whole warp) --------------
    // eph: bit i = parity of the number of uses of ring barrier i so far; used: barriers ever armed
    uint32_t eph = 0, used = 0, unit_phase = 0, res_armed = 0;
    bool ok = true;
    for (int unit = cluster_id; ok; unit += n_clusters) {
      const ResUnit w = decode_res(p, unit, split);
      if (!w.valid) break;
      if (w.rows == 0) continue;                       // empty expert: the epilogue writes zeros
      // resident operand: wait until the previous unit's MMAs are done with it, then load
      ok = warp_wait(false, bfree, unit_phase ^ 1, abort_flag, p.fault, 31);
      if (!ok) break;
      const int ns = (w.rows + kWBK - 1) / kWBK;
      if (ns > RES) {                                  // the host bounds this; never index past the buffer
        if (lane == 0) { *abort_flag = 1; atomicCAS(p.fault, 0, 35); }
        ok = false;
        break;
      }
      if (leader && lane == 0) mbar_expect_tx(bfull, 2u * (uint32_t)ns * kResStageBytes);
      ++res_armed;
      __syncwarp();
      {
        // boxes 2s and 2s + 1 of the resident operand are issued by lanes 2s and 2s + 1
        const int qh = w.q0 + 128 * (int)rank;         // this CTA's half of the columns
        const uint32_t bar = bfull & kPeerMask;
        const int s = lane >> 1;
        if (s < ns)
          tma2_load_2d(res_base + s * kResStageBytes + (lane & 1) * kBoxBytes, &tmap_b, bar,
                       qh + 64 * (lane & 1), w.row0 + s * kWBK);
      }
      // streamed operand: every p-block walks the expert's stages.  The ring takes the stages the
      // resident operand leaves (it is empty here: the wait on bfree above saw every MMA retire)
      const int ring = kResTotalStages - ns;
      const uint32_t ring_base = res_base + ns * kResStageBytes;
      int stage = 0;
      for (int pb = w.pb0; pb < w.pb1 && ok; ++pb) {
        const int ph = pb * 256 + 128 * (int)rank + 64 * (lane & 1);     // this lane's 64 output rows
        for (int s = 0; s < ns && ok; ++s) {
          ok = warp_wait(false, empty0 + 8 * stage, ((eph >> stage) & 1u) ^ 1u, abort_flag, p.fault, 32);
          if (ok) {
            const uint32_t bar = (full0 + 8 * stage) & kPeerMask;
            const uint32_t sa = ring_base + stage * kResStageBytes;
            if (leader && lane == 0) mbar_expect_tx(full0 + 8 * stage, 2u * kResStageBytes);
            if (lane < 2) tma2_load_2d(sa + lane * kBoxBytes, &tmap_a, bar, ph, w.row0 + s * kWBK);
            eph ^= 1u << stage;
            used |= 1u << stage;
            if (++stage == ring) stage = 0;
          }
        }
      }
      unit_phase ^= 1;
    }
    if (leader && lane == 0 && *abort_flag) {
      const uint64_t deadline = globaltimer_ns() + 200000000ull;
      for (int i = 0; i < STAGES; ++i)               // the last phase armed on each ring barrier
        if ((used >> i) & 1u) mbar_drain(full0 + 8 * i, ((eph >> i) & 1u) ^ 1u, deadline);
      if (res_armed > 0) mbar_drain(bfull, (res_armed - 1) & 1u, globaltimer_ns() + 200000000ull);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA only) -----------------------
    if (lane == 0 && leader) {
      int acc = 0;
      uint32_t fph = 0, acc_phase = 0, unit_phase = 0;      // fph: as eph in the producer
      bool ok = true;
      for (int unit = cluster_id; ok; unit += n_clusters) {
        const ResUnit w = decode_res(p, unit, split);
        if (!w.valid) break;
        if (w.rows == 0) continue;
        const int ns = (w.rows + kWBK - 1) / kWBK;
        if (ns > RES) break;                          // the producer has raised the fault
        if (!(ok = mbar_wait(bfull, unit_phase, abort_flag, p.fault, 33))) break;
        tcgen05_fence_after();
        const int ring = kResTotalStages - ns;
        const uint32_t ring_base = res_base + ns * kResStageBytes;
        int stage = 0;
        for (int pb = w.pb0; pb < w.pb1 && ok; ++pb) {
          if (!(ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.fault, 12))) break;
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * 256;
          for (int s = 0; s < ns; ++s) {
            const int ksteps = res_ksteps(w.rows, s);
            const int st_a = stage;
            if (!(ok = mbar_wait(full0 + 8 * st_a, (fph >> st_a) & 1u, abort_flag, p.fault, 13))) break;
            const uint32_t sa = ring_base + st_a * kResStageBytes;
            const uint32_t sb = res_base + s * kResStageBytes;
            tcgen05_fence_after();
            // a full stage is straight-line code: a branch between the MMAs slows their issue
            if (ksteps == kWBK / kUmmaK) {
#pragma unroll
              for (int ks = 0; ks < kWBK / kUmmaK; ++ks)
                tcgen05_mma2_bf16(d_tmem, make_desc(sa + ks * (kUmmaK * 128), kBoxBytes, 1024),
                                  make_desc(sb + ks * (kUmmaK * 128), kBoxBytes, 1024), kIdesc,
                                  (s == 0 && ks == 0) ? 0u : 1u);
            } else {
              for (int ks = 0; ks < ksteps; ++ks)
                tcgen05_mma2_bf16(d_tmem, make_desc(sa + ks * (kUmmaK * 128), kBoxBytes, 1024),
                                  make_desc(sb + ks * (kUmmaK * 128), kBoxBytes, 1024), kIdesc,
                                  (s == 0 && ks == 0) ? 0u : 1u);
            }
            tcgen05_commit2(empty0 + 8 * st_a);
            fph ^= 1u << st_a;
            stage = st_a + 1 == ring ? 0 : st_a + 1;
          }
          if (!ok) break;
          tcgen05_commit2(tfull0 + 8 * acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (!ok) break;
        tcgen05_commit2(bfree);                       // the resident operand may be replaced
        unit_phase ^= 1;
      }
      if (*abort_flag) {
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
    bool ok = true;
    for (int unit = cluster_id; ok; unit += n_clusters) {
      const ResUnit w = decode_res(p, unit, split);
      if (!w.valid) break;
      const int slot = p.slot.s[p.e_begin + w.el];
      const bool empty = w.rows == 0;
      for (int pb = w.pb0; pb < w.pb1; ++pb) {
        const int lrow = quarter * 32 + lane;
        const int64_t obase = ((int64_t)slot * p.P + pb * 256 + 128 * (int)rank + lrow) * p.N + w.q0;
        constexpr int NSTEPS = 256 / 4 / kEpiStep;
        uint32_t pre[NSTEPS][8];
        epilogue_prefetch<EV, NSTEPS>(p, obase, nullptr, nullptr, cq * 64, pre);
        if (!empty) {
          if (!(ok = warp_wait(false, tfull0 + 8 * acc, acc_phase, abort_flag, p.fault, 14))) break;
          tcgen05_fence_after();
        }
        using Ev = EvTraits<EV>;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
        if (EV == EV_WGRAD)
          epilogue_lines<NSTEPS>(p.out0, obase - (int64_t)lane * p.N, p.N, taddr, empty, cq * 64,
                                 store_strip[ew]);
        else
          epilogue_loop<Ev::epi, Ev::act, Ev::gbwd, Ev::bias, Ev::accum, NSTEPS>(
              p, taddr, empty, true, p.out0, obase, nullptr, cq * 64, pre, nullptr);
        if (!empty) {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster((tempty0 + 8 * acc) & kPeerMask);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  }

  tcgen05_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols) : "memory");
  }
}
