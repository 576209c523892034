// Internal interface between the FFN orchestration (ffn.cu) and the two grouped-GEMM back
// ends: gemm_simt.cu (fp32 and bf16 on CUDA cores, exact fp32 accumulation in a fixed order;
// the fp32 layer runs on it) and gemm_tc.cu (bf16 on tcgen05 tensor cores, the performance
// path).
#pragma once
#include "common.cuh"

namespace mole {

constexpr int kMaxLocalExperts = 256;
struct SlotMap {
  int16_t s[kMaxLocalExperts];   // local expert -> slot in the batched weight / grad array
};

// Row-grouped GEMM:  out[r, n] = epilogue( sum_k A[r, k] * W_e(k, n) )  for every scheduled
// 128-row tile; e = tile_expert.  W_e = W + slot(e) * w_expert_stride is [N, K] (w_nk = 1:
// FC1, dX2) or [K, N] (w_nk = 0: FC2, dX); both views of the reference's [F, M] weights.
struct RowGemmArgs {
  const void* A;        // [rows, K]
  const void* W;        // [n_slots, F, M]
  int64_t w_expert_stride;
  int n_slots;
  int w_nk;
  int N, K;
  const void* bias;     // [n_slots, N] or null
  const void* aux;      // [rows, N]  (EPI_DACT: pre-activation)
  void* out0;           // [rows, N]
  void* out1;           // [rows, N]  (EPI_FC1: activation)
  int64_t total_rows;   // extent of the row buffers
  int epi, act, gelu_bwd;
  int e_begin, n_experts;   // experts covered by the schedule
  int single_cta;           // tensor cores: keep to the one-CTA kernel (A/B comparisons)
  int panel;                // tensor cores: every expert's rows are one contiguous run and the panel
                            // kernel may take the launch (outputs in place, no fused combine)
  int max_rows_per_expert;  // bound on an expert's rows (sizes the panel kernel's stages)
  float* colsum_ws;         // dX2 on the panel kernel: room for partial column sums of the output
                            // (tc_panel_colsum_bytes), or null: no fused column sums
  const int32_t* rowmap;    // tensor cores, FC2 / dX: scatter output rows (-1 = drop), or null
  PeerMap peers;            // with rowmap: the scattered rows go to their source ranks (n > 0)
  int peer_Cs;              // rows per chunk of the receive buffers
  // FC2 with the gate-weighted combine in its epilogue (c_y != null): y[t] += gates[pair] * out[row]
  const int32_t* c_perm;
  const int32_t* c_offsets;
  const int32_t* c_counts;
  const float* c_gates;
  void* c_y;
  int c_k, c_Cs;
  Schedule sched;
  SlotMap wslot;
};

// Weight-gradient GEMM:  out_e[p, q] (+)= sum_{r in tiles of e} A[r, p] * B[r, q]
struct WgradArgs {
  const void* A;        // [rows, P]
  const void* B;        // [rows, Q]
  int P, Q;
  void* out;            // [n_slots, P, Q]
  int n_slots;
  int64_t total_rows;
  int accumulate;
  int e_begin, n_experts;
  int single_cta;
  int resident;               // tensor cores: the resident-operand kernel may take the launch
  int max_tiles_per_expert;   // bound on an expert's 128-row tiles (sizes the resident operand)
  Schedule sched;
  SlotMap gslot;
};

// Column sums per expert: out[slot(e), n] (+)= sum_{r in tiles of e} A[r, n]
struct ColsumArgs {
  const void* A;
  int N;
  void* out;            // [n_slots, N]
  int accumulate;
  int e_begin, n_experts;
  Schedule sched;
  SlotMap gslot;
};

int build_schedule(const int32_t* counts, int L, int n_src, int Cs, int e_begin, int e_end,
                   Schedule s, cudaStream_t st);
int build_schedule_compact(const int32_t* counts, int L, int n_src, int Cs, int e_begin, int e_end,
                           Schedule s, cudaStream_t st);
int compact_gather(int dtype, const void* src, const int32_t* counts, int L, int n_src, int Cs,
                   int e_begin, int e_end, int width, void* dst, int32_t* rowmap, cudaStream_t st);
int64_t schedule_bytes(int L, int n_src, int Cs);
Schedule carve_schedule(void* ws, int L, int n_src, int Cs);

int simt_row_gemm(int dtype, const RowGemmArgs& a, cudaStream_t st);
int simt_wgrad(int dtype, const WgradArgs& a, cudaStream_t st);
int colsum(int dtype, const ColsumArgs& a, cudaStream_t st);

int tc_row_gemm(const RowGemmArgs& a, cudaStream_t st);     // bf16 only
int tc_wgrad(const WgradArgs& a, cudaStream_t st);          // bf16 only
// Column sums of dX1 fused into the dX2 launch (panel kernel only): whether tc_row_gemm(a) leaves
// the partial sums in a.colsum_ws, their size, and the fixed-order reduction into out[slot, N].
bool tc_panel_colsum(const RowGemmArgs& a);
int64_t tc_panel_colsum_bytes(int n_experts, int max_rows_per_expert, int N);
int tc_panel_colsum_reduce(const RowGemmArgs& a, const SlotMap& gslot, int accumulate, void* out,
                           cudaStream_t st);
bool tc_supported(int M, int F);

// scalar epilogue shared by both back ends
struct EpiOut { float v0, v1; };
__device__ __forceinline__ EpiOut epilogue_apply(int epi, float acc, float bias, float aux, int act,
                                                 int gelu_bwd) {
  EpiOut o;
  o.v1 = 0.f;
  switch (epi) {
    case EPI_FC1:  o.v0 = acc + bias; o.v1 = act_fwd(o.v0, act); break;
    case EPI_BIAS: o.v0 = acc + bias; break;
    case EPI_DACT: o.v0 = acc * act_grad(aux, act, gelu_bwd); break;
    default:       o.v0 = acc; break;
  }
  return o;
}

}  // namespace mole
