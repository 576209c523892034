// Expert FFN forward / backward over capacity-strided rows: tile schedule + grouped GEMMs.
//
// forward  (MOLE/cpp/core.cpp:350-353):  x1 = x W1^T + b1;  h = act(x1);  out = h W2 + b2
// backward (MOLE/cpp/core.cpp:388-412):  gW2 = h^T dO;  dX1 = (dO W2^T) * act'(x1);  gb2 = sum dO;
//                                        gW1 = dX1^T x;  gb1 = sum dX1;  dX = dX1 W1
// with "=" or "+=" into the gradients (core.cpp:274-316).  The reference runs these on the
// capacity-padded [B, W*C, .] tensors after a permute+contiguous re-layout; here the schedule
// points the GEMMs at the (source rank, expert) chunks where they lie and skips empty tiles.
#include "gemm.cuh"

namespace mole {

static int check_desc(const mole_ffn_desc* d) {
  MOLE_REQUIRE(d != nullptr, "desc is null");
  MOLE_REQUIRE(d->dtype == MOLE_F32 || d->dtype == MOLE_BF16, "dtype %d", d->dtype);
  MOLE_REQUIRE(d->act == MOLE_ACT_GELU || d->act == MOLE_ACT_RELU, "act %d", d->act);
  MOLE_REQUIRE(d->M > 0 && d->F > 0 && d->M % 64 == 0 && d->F % 64 == 0,
               "M=%d and F=%d must be positive multiples of 64", d->M, d->F);
  MOLE_REQUIRE(d->L >= 1 && d->L <= kMaxLocalExperts, "L=%d not in [1,%d]", d->L, kMaxLocalExperts);
  MOLE_REQUIRE(d->n_src >= 1, "n_src=%d", d->n_src);
  MOLE_REQUIRE(d->Cs > 0 && d->Cs % kTileRows == 0, "Cs=%d must be a positive multiple of 128", d->Cs);
  MOLE_REQUIRE(0 <= d->e_begin && d->e_begin <= d->e_end && d->e_end <= d->L,
               "expert range [%d,%d) outside [0,%d)", d->e_begin, d->e_end, d->L);
  MOLE_REQUIRE(d->n_slots >= 1 && d->n_slots <= 32767, "n_slots=%d", d->n_slots);
  MOLE_REQUIRE(d->n_grad_slots >= 0 && d->n_grad_slots <= 32767, "n_grad_slots=%d", d->n_grad_slots);
  MOLE_REQUIRE((int64_t)d->L * d->n_src * d->Cs < ((int64_t)1 << 31), "row index overflows int32");
  if (d->dtype == MOLE_BF16 && d->backend != 1 && !tc_supported(d->M, d->F))
    return fail(MOLE_ERR_UNSUPPORTED,
                "bf16 tensor-core path needs M and F to be multiples of 128 (M=%d F=%d)", d->M, d->F);
  return MOLE_OK;
}

static int fill_slots(SlotMap& m, const mole_ffn_desc* d, const int32_t* host_map, int n_slots) {
  for (int l = 0; l < kMaxLocalExperts; ++l) m.s[l] = 0;
  for (int l = d->e_begin; l < d->e_end; ++l) {
    const int s = host_map ? host_map[l] : l;
    MOLE_REQUIRE(s >= 0 && s < n_slots, "slot %d of expert %d outside [0,%d)", s, l, n_slots);
    m.s[l] = (int16_t)s;
  }
  return MOLE_OK;
}

static bool use_tc(const mole_ffn_desc* d) { return d->dtype == MOLE_BF16 && d->backend != 1; }
// CTA pairs (cta_group::2) pay off when an expert has many row tiles: the pair halves the
// weight bytes read through L2 per product, but an odd tile count idles half a pair.  With few
// tiles per expert the GEMMs are bound by HBM (weights are read once whatever the tile shape)
// and the one-CTA kernel's finer granularity wins; measured crossover is around a dozen tiles.
static int single_cta(const mole_ffn_desc* d) {
  if (d->backend == 2) return 1;
  if (d->backend == 3) return 0;
  return d->n_src * (d->Cs / kTileRows) < 12;
}
static bool compacting(const mole_ffn_desc* d);
// The panel kernel (weights on the M side of the MMA, an expert's rows on the N side in steps of
// 16) needs every expert's rows in one run: one source rank, or the compacted layout.
static bool contiguous_rows(const mole_ffn_desc* d) { return d->n_src == 1 || compacting(d); }
// Row GEMMs: measured 3-12 % faster than the tile kernels at a few hundred rows per expert, ragged
// or not (a short last tile costs the tile kernels a whole one); with many tiles per expert the
// CTA-pair tile kernel does the same work per staged byte and keeps the lighter epilogue.
static int panel_ok(const mole_ffn_desc* d) {
  if (!contiguous_rows(d)) return 0;
  return d->backend == 4 || (d->backend == 0 && d->n_src * d->Cs <= 1024);
}
// The resident-operand weight gradient: same requirement; measured faster than the tile kernels
// wherever an expert's rows fit its shared-memory budget (the launch falls back beyond it).
static int resident_ok(const mole_ffn_desc* d) {
  return (d->backend == 0 || d->backend == 4) && contiguous_rows(d);
}

// With several source ranks per expert the tensor-core path first packs each expert's rows of
// all sources into one run (gemm_simt.cu, "per-expert compaction"): x1, h and dX1 then live in that
// layout, FC2 / dX scatter their output rows back to the (source, expert) chunks.  `desc.compact`
// = 2 switches it off (comparisons).
static bool compacting(const mole_ffn_desc* d) { return use_tc(d) && d->n_src > 1 && d->compact != 2; }
// compact == 3: the caller's row buffers (x, dout) already are in the packed layout -- the senders
// of the push-style exchange put every row at its final place -- so nothing is gathered: the
// call only builds the row map and zeroes the pad rows of those buffers, in place.
static bool prepacked(const mole_ffn_desc* d) { return compacting(d) && d->compact == 3; }

struct Workspace {
  Schedule sched;
  int32_t* rowmap;   // [rows_total]
  void* buf_a;       // [rows_total, M]
  void* buf_b;       // [rows_total, M]
  float* colsum;     // partial column sums of dX1 from the dX2 launch (panel kernel), or null
};
// Column sums of dX1 (the FC1 bias gradient) come out of the dX2 launch when the panel kernel
// takes it (its epilogue threads each own one feature and walk down the rows anyway) or the
// CTA-pair tile kernel (many rows per expert: the epilogue is hidden behind the main loop).
static bool fused_colsum(const mole_ffn_desc* d) {
  return use_tc(d) && d->F % 256 == 0 && (panel_ok(d) || !single_cta(d));
}
static int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }
static int64_t workspace_bytes_of(const mole_ffn_desc* d) {
  int64_t b = align256(schedule_bytes(d->L, d->n_src, d->Cs));
  if (compacting(d)) {
    const int64_t rows = (int64_t)d->L * d->n_src * d->Cs;
    b += align256(rows * 4);
    if (!prepacked(d)) b += 2 * align256(rows * d->M * 2);
  }
  if (fused_colsum(d)) b += align256(tc_panel_colsum_bytes(d->L, d->n_src * d->Cs, d->F));
  return b;
}
static Workspace carve_workspace(const mole_ffn_desc* d, void* ws) {
  Workspace w{};
  w.sched = carve_schedule(ws, d->L, d->n_src, d->Cs);
  char* p = static_cast<char*>(ws) + align256(schedule_bytes(d->L, d->n_src, d->Cs));
  if (compacting(d)) {
    const int64_t rows = (int64_t)d->L * d->n_src * d->Cs;
    w.rowmap = reinterpret_cast<int32_t*>(p);
    p += align256(rows * 4);
    if (!prepacked(d)) {
      w.buf_a = p;
      p += align256(rows * d->M * 2);
      w.buf_b = p;
      p += align256(rows * d->M * 2);
    }
  }
  if (fused_colsum(d)) w.colsum = reinterpret_cast<float*>(p);
  return w;
}

static int row_gemm(const mole_ffn_desc* d, const RowGemmArgs& a, cudaStream_t st) {
  return use_tc(d) ? tc_row_gemm(a, st) : simt_row_gemm(d->dtype, a, st);
}
static int wgrad(const mole_ffn_desc* d, const WgradArgs& a, cudaStream_t st) {
  return use_tc(d) ? tc_wgrad(a, st) : simt_wgrad(d->dtype, a, st);
}

}  // namespace mole

using namespace mole;

extern "C" int mole_ffn_workspace_bytes(const mole_ffn_desc* d, int64_t* bytes) {
  if (int rc = check_desc(d)) return rc;
  MOLE_REQUIRE(bytes != nullptr, "bytes is null");
  *bytes = workspace_bytes_of(d);
  return MOLE_OK;
}

// Push-style return exchange: the scattered output rows of FC2 (forward) and dX (backward) go
// straight into the source ranks' receive buffers.  Needs the packed path (its row map).
static int peers_for_ffn(const mole_ffn_desc* d, void* const* peer_rows, int rank, PeerMap& pm) {
  MOLE_REQUIRE(compacting(d), "peer output needs the bf16 tensor-core path with n_src > 1");
  MOLE_REQUIRE(peer_rows != nullptr, "null peer table");
  MOLE_REQUIRE(d->n_src <= kMaxPeers, "at most %d source ranks", kMaxPeers);
  MOLE_REQUIRE(rank >= 0 && rank < d->n_src, "rank %d outside the %d source ranks", rank, d->n_src);
  pm = PeerMap{};
  for (int q = 0; q < d->n_src; ++q) {
    MOLE_REQUIRE(peer_rows[q] != nullptr, "null buffer for peer %d", q);
    pm.base[q] = peer_rows[q];
  }
  pm.n = d->n_src;
  pm.rank = rank;
  pm.L = d->L;
  return MOLE_OK;
}

struct CombineArgs {
  const int32_t* offsets;
  const int32_t* perm;
  const float* gates;
  int k;
  void* y;
};
static int ffn_fwd_impl(const mole_ffn_desc* d, const int32_t* counts,
                        const int32_t* slot_of_expert, const void* x, const void* w1,
                        const void* b1, const void* w2, const void* b2, void* x1, void* h,
                        void* out, const PeerMap* peers, const CombineArgs* comb, void* workspace,
                        int64_t workspace_bytes, void* stream);

extern "C" int mole_ffn_fwd(const mole_ffn_desc* d, const int32_t* counts,
                            const int32_t* slot_of_expert, const void* x, const void* w1,
                            const void* b1, const void* w2, const void* b2, void* x1, void* h,
                            void* out, void* workspace, int64_t workspace_bytes, void* stream) {
  MOLE_REQUIRE(out != nullptr, "null pointer argument");
  return ffn_fwd_impl(d, counts, slot_of_expert, x, w1, b1, w2, b2, x1, h, out, nullptr, nullptr,
                      workspace, workspace_bytes, stream);
}

// FC2's epilogue also adds gates[pair] * row into y[token] (bf16 reductions at L2; the caller
// zeroes y first): the combine needs no pass of its own over the expert outputs.  The rows are
// still stored, backward reads them for the gate gradient.
extern "C" int mole_ffn_fwd_combine(const mole_ffn_desc* d, const int32_t* counts,
                                    const int32_t* slot_of_expert, const void* x, const void* w1,
                                    const void* b1, const void* w2, const void* b2, void* x1,
                                    void* h, void* out, const int32_t* offsets,
                                    const int32_t* perm, const float* gates, int32_t k, void* y,
                                    void* workspace, int64_t workspace_bytes, void* stream) {
  if (int rc = check_desc(d)) return rc;
  MOLE_REQUIRE(out && offsets && perm && gates && y, "null pointer argument");
  MOLE_REQUIRE(k >= 1 && k <= 2, "the fused combine covers top-1 and top-2 (k=%d): with more addends "
               "per token the order of the reductions would show in the result", k);
  if (!(use_tc(d) && d->n_src == 1 && single_cta(d)))
    return fail(MOLE_ERR_UNSUPPORTED, "the fused combine needs bf16 on the one-CTA tensor-core kernel "
                "(fewer than 12 row tiles per expert) and one source rank");
  CombineArgs c{offsets, perm, gates, k, y};
  return ffn_fwd_impl(d, counts, slot_of_expert, x, w1, b1, w2, b2, x1, h, out, nullptr, &c,
                      workspace, workspace_bytes, stream);
}

extern "C" int mole_ffn_fwd_peer(const mole_ffn_desc* d, const int32_t* counts,
                                 const int32_t* slot_of_expert, const void* x, const void* w1,
                                 const void* b1, const void* w2, const void* b2, void* x1, void* h,
                                 void* const* peer_out, int32_t rank, void* workspace,
                                 int64_t workspace_bytes, void* stream) {
  if (int rc = check_desc(d)) return rc;
  PeerMap pm;
  if (int rc = peers_for_ffn(d, peer_out, rank, pm)) return rc;
  return ffn_fwd_impl(d, counts, slot_of_expert, x, w1, b1, w2, b2, x1, h, nullptr, &pm, nullptr,
                      workspace, workspace_bytes, stream);
}

static int ffn_fwd_impl(const mole_ffn_desc* d, const int32_t* counts,
                        const int32_t* slot_of_expert, const void* x, const void* w1,
                        const void* b1, const void* w2, const void* b2, void* x1, void* h,
                        void* out, const PeerMap* peers, const CombineArgs* comb, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  if (int rc = check_desc(d)) return rc;
  MOLE_REQUIRE(counts && x && w1 && b1 && w2 && b2 && x1 && h && (out || peers) && workspace,
               "null pointer argument");
  MOLE_REQUIRE(workspace_bytes >= workspace_bytes_of(d), "workspace too small");
  if (d->e_begin == d->e_end) return MOLE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Workspace wk = carve_workspace(d, workspace);
  const Schedule s = wk.sched;
  const bool compact = compacting(d);
  if (compact) {
    if (int rc = build_schedule_compact(counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, s, st)) return rc;
    if (prepacked(d)) {
      if (int rc = compact_gather(d->dtype, nullptr, counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end,
                                  d->M, const_cast<void*>(x), wk.rowmap, st)) return rc;
    } else {
      if (int rc = compact_gather(d->dtype, x, counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, d->M,
                                  wk.buf_a, wk.rowmap, st)) return rc;
      x = wk.buf_a;
    }
  } else {
    if (int rc = build_schedule(counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, s, st)) return rc;
  }

  RowGemmArgs a{};
  if (int rc = fill_slots(a.wslot, d, slot_of_expert, d->n_slots)) return rc;
  a.sched = s;
  a.w_expert_stride = (int64_t)d->F * d->M;
  a.n_slots = d->n_slots;
  a.total_rows = (int64_t)d->L * d->n_src * d->Cs;
  a.act = d->act;
  a.gelu_bwd = d->gelu_bwd;
  a.e_begin = d->e_begin;
  a.n_experts = d->e_end - d->e_begin;
  a.single_cta = single_cta(d);
  a.panel = panel_ok(d); a.max_rows_per_expert = d->n_src * d->Cs;
  // FC1: [rows, M] x W1_e^T ([F, M] read as [N=F][K=M])
  a.A = x; a.W = w1; a.w_nk = 1; a.N = d->F; a.K = d->M; a.bias = b1; a.aux = nullptr;
  a.out0 = x1; a.out1 = h; a.epi = EPI_FC1;
  if (int rc = row_gemm(d, a, st)) return rc;
  // FC2: [rows, F] x W2_e ([F, M] read as [K=F][N=M])
  a.A = h; a.W = w2; a.w_nk = 0; a.N = d->M; a.K = d->F; a.bias = b2;
  a.out0 = out; a.out1 = nullptr; a.epi = EPI_BIAS;
  a.rowmap = compact ? wk.rowmap : nullptr;          // back to the (source, expert) chunks
  if (peers) { a.peers = *peers; a.peer_Cs = d->Cs; }
  if (comb) {
    a.c_perm = comb->perm; a.c_offsets = comb->offsets; a.c_counts = counts; a.c_gates = comb->gates;
    a.c_y = comb->y; a.c_k = comb->k; a.c_Cs = d->Cs;
  }
  return row_gemm(d, a, st);
}

static int ffn_bwd_impl(const mole_ffn_desc* d, const int32_t* counts,
                        const int32_t* slot_of_expert, const int32_t* grad_slot_of_expert,
                        const void* dout, const void* x, const void* x1, const void* h,
                        const void* w1, const void* w2, void* dx1, void* dx, const PeerMap* peers,
                        void* gw1, void* gb1, void* gw2, void* gb2, void* workspace,
                        int64_t workspace_bytes, void* stream);

extern "C" int mole_ffn_bwd(const mole_ffn_desc* d, const int32_t* counts,
                            const int32_t* slot_of_expert, const int32_t* grad_slot_of_expert,
                            const void* dout, const void* x, const void* x1, const void* h,
                            const void* w1, const void* w2, void* dx1, void* dx, void* gw1,
                            void* gb1, void* gw2, void* gb2, void* workspace,
                            int64_t workspace_bytes, void* stream) {
  return ffn_bwd_impl(d, counts, slot_of_expert, grad_slot_of_expert, dout, x, x1, h, w1, w2, dx1,
                      dx, nullptr, gw1, gb1, gw2, gb2, workspace, workspace_bytes, stream);
}

extern "C" int mole_ffn_bwd_peer(const mole_ffn_desc* d, const int32_t* counts,
                                 const int32_t* slot_of_expert,
                                 const int32_t* grad_slot_of_expert, const void* dout,
                                 const void* x, const void* x1, const void* h, const void* w1,
                                 const void* w2, void* dx1, void* const* peer_dx, int32_t rank,
                                 void* gw1, void* gb1, void* gw2, void* gb2, void* workspace,
                                 int64_t workspace_bytes, void* stream) {
  if (int rc = check_desc(d)) return rc;
  PeerMap pm;
  if (int rc = peers_for_ffn(d, peer_dx, rank, pm)) return rc;
  return ffn_bwd_impl(d, counts, slot_of_expert, grad_slot_of_expert, dout, x, x1, h, w1, w2, dx1,
                      nullptr, &pm, gw1, gb1, gw2, gb2, workspace, workspace_bytes, stream);
}

static int ffn_bwd_impl(const mole_ffn_desc* d, const int32_t* counts,
                        const int32_t* slot_of_expert, const int32_t* grad_slot_of_expert,
                        const void* dout, const void* x, const void* x1, const void* h,
                        const void* w1, const void* w2, void* dx1, void* dx, const PeerMap* peers,
                        void* gw1, void* gb1, void* gw2, void* gb2, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  if (int rc = check_desc(d)) return rc;
  MOLE_REQUIRE(counts && dout && x && x1 && h && w1 && w2 && dx1 && gw1 && gb1 && gw2 && gb2 &&
               workspace, "null pointer argument");
  MOLE_REQUIRE(workspace_bytes >= workspace_bytes_of(d), "workspace too small");
  if (d->e_begin == d->e_end) return MOLE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Workspace wk = carve_workspace(d, workspace);
  const Schedule s = wk.sched;
  const bool compact = compacting(d);
  if (compact) {      // x1, h come compacted from forward; x and dout are packed the same way here
    if (int rc = build_schedule_compact(counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, s, st)) return rc;
    if (prepacked(d)) {      // x was prepared by forward; dout's pad rows are zeroed here
      if (int rc = compact_gather(d->dtype, nullptr, counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end,
                                  d->M, const_cast<void*>(dout), wk.rowmap, st)) return rc;
    } else {
      if (int rc = compact_gather(d->dtype, x, counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, d->M,
                                  wk.buf_a, wk.rowmap, st)) return rc;
      if (int rc = compact_gather(d->dtype, dout, counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end,
                                  d->M, wk.buf_b, nullptr, st)) return rc;
      x = wk.buf_a;
      dout = wk.buf_b;
    }
  } else {
    if (int rc = build_schedule(counts, d->L, d->n_src, d->Cs, d->e_begin, d->e_end, s, st)) return rc;
  }
  const int64_t total_rows = (int64_t)d->L * d->n_src * d->Cs;
  const int n_experts = d->e_end - d->e_begin;

  SlotMap wslot, gslot;
  const int n_grad_slots = d->n_grad_slots > 0 ? d->n_grad_slots : d->n_slots;
  if (int rc = fill_slots(wslot, d, slot_of_expert, d->n_slots)) return rc;
  if (int rc = fill_slots(gslot, d, grad_slot_of_expert, n_grad_slots)) return rc;

  WgradArgs g{};
  g.sched = s; g.gslot = gslot; g.n_slots = n_grad_slots; g.total_rows = total_rows;
  g.accumulate = d->accumulate; g.e_begin = d->e_begin; g.n_experts = n_experts;
  g.P = d->F; g.Q = d->M; g.single_cta = single_cta(d);
  g.resident = resident_ok(d); g.max_tiles_per_expert = d->n_src * (d->Cs / kTileRows);
  ColsumArgs c{};
  c.sched = s; c.gslot = gslot; c.accumulate = d->accumulate; c.e_begin = d->e_begin;
  c.n_experts = n_experts;

  // gW2 = h^T dO
  g.A = h; g.B = dout; g.out = gw2;
  if (int rc = wgrad(d, g, st)) return rc;
  // dX1 = (dO W2^T) * act'(x1):  W2_e read as [N=F][K=M]
  RowGemmArgs a{};
  a.sched = s; a.wslot = wslot; a.w_expert_stride = (int64_t)d->F * d->M; a.n_slots = d->n_slots;
  a.total_rows = total_rows; a.act = d->act; a.gelu_bwd = d->gelu_bwd;
  a.e_begin = d->e_begin; a.n_experts = n_experts; a.single_cta = single_cta(d);
  a.panel = panel_ok(d); a.max_rows_per_expert = d->n_src * d->Cs;
  a.A = dout; a.W = w2; a.w_nk = 1; a.N = d->F; a.K = d->M; a.bias = nullptr; a.aux = x1;
  a.out0 = dx1; a.out1 = nullptr; a.epi = EPI_DACT;
  a.colsum_ws = wk.colsum;
  const bool gb1_fused = use_tc(d) && tc_panel_colsum(a);
  if (int rc = row_gemm(d, a, st)) return rc;
  // gb1 = sum_rows dX1: left as partial sums by the launch above, or by a pass over dX1 below
  if (gb1_fused) {
    if (int rc = tc_panel_colsum_reduce(a, gslot, d->accumulate, gb1, st)) return rc;
  }
  a.colsum_ws = nullptr;
  // gb2 = sum_rows dO
  c.A = dout; c.N = d->M; c.out = gb2;
  if (int rc = colsum(d->dtype, c, st)) return rc;
  // gW1 = dX1^T x
  g.A = dx1; g.B = x; g.out = gw1;
  if (int rc = wgrad(d, g, st)) return rc;
  // gb1 = sum_rows dX1
  if (!gb1_fused) {
    c.A = dx1; c.N = d->F; c.out = gb1;
    if (int rc = colsum(d->dtype, c, st)) return rc;
  }
  // dX = dX1 W1:  W1_e read as [K=F][N=M]
  if (dx != nullptr || peers != nullptr) {
    a.A = dx1; a.W = w1; a.w_nk = 0; a.N = d->M; a.K = d->F; a.bias = nullptr; a.aux = nullptr;
    a.out0 = dx; a.out1 = nullptr; a.epi = EPI_STORE;
    a.rowmap = compact ? wk.rowmap : nullptr;
    if (peers) { a.peers = *peers; a.peer_Cs = d->Cs; }
    if (int rc = row_gemm(d, a, st)) return rc;
  }
  return MOLE_OK;
}
