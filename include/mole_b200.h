/*
 * mole_b200 -- C ABI of the B200-native (sm_100a) MoE-layer hot path.
 *
 * This library replaces the pybind11 module `core` of atc23-101/MOLE
 * (MOLE/cpp/core.cpp:1347-1469) and the third-party routing / dispatch / combine
 * kernels the reference layer calls (MOLE/moe/layer.py:445-449, 457-458).
 *
 * Conventions
 *   - every entry point returns 0 (MOLE_OK) or a negative mole_status; nothing
 *     throws, exits or aborts.  mole_last_error_string() describes the last failure
 *     on the calling thread.
 *   - all tensor arguments are raw device pointers (host pointers only where the
 *     name says "host"); the caller owns every buffer and keeps it alive until the
 *     stream work has completed.  `stream` is a cudaStream_t passed as void*.
 *   - the library allocates nothing on the data path except where stated.
 *   - `dtype` selects the element type of activations and weights (MOLE_F32 or
 *     MOLE_BF16); routing integers are int32, scores / gate weights are fp32.
 *
 * Row layout shared by dispatch, FFN and combine ("capacity-strided rows"):
 *   a row buffer is [n_chunks][Cs][width]; chunk c holds the rows of one
 *   (source rank, expert) pair, Cs = mole_capacity_stride(C) is the capacity
 *   rounded up to 128 rows; counts[c] <= C rows are valid, rows up to the next
 *   multiple of 128 are zero, rows beyond that are never read or written.
 *   On a single GPU chunk index == expert index, so with C % 128 == 0 this is the
 *   reference's dispatched tensor [E, C, M] (MOLE/cpp/core.cpp:993-995).
 */
#ifndef MOLE_B200_H_
#define MOLE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  MOLE_OK = 0,
  MOLE_ERR_INVALID = -1,      /* bad argument (size, alignment, null pointer)          */
  MOLE_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed                   */
  MOLE_ERR_NCCL = -3,         /* an NCCL call failed                                   */
  MOLE_ERR_UNSUPPORTED = -4,  /* shape / dtype outside what the kernels cover          */
  MOLE_ERR_STATE = -5,        /* call order violated (pool / prefetch stack)           */
  MOLE_ERR_DEVICE = -6        /* a kernel recorded a fault (bounded wait ran out, ...)  */
} mole_status;

typedef enum { MOLE_F32 = 0, MOLE_BF16 = 1 } mole_dtype;
typedef enum { MOLE_ACT_GELU = 0, MOLE_ACT_RELU = 1 } mole_act;
/* derivative used for GELU in backward: exact (at::gelu_backward, the #else branch at
 * MOLE/cpp/core.cpp:396) or the tanh approximation of MOLE/cpp/gelu.cu:3-14 */
typedef enum { MOLE_GELU_BWD_EXACT = 0, MOLE_GELU_BWD_TANH = 1 } mole_gelu_bwd;

int mole_version(void);
const char* mole_last_error_string(void);
/* capacity rounded up to the 128-row tile of the grouped GEMM */
int64_t mole_capacity_stride(int64_t capacity);
/* reads and clears the device-side fault word written by kernels whose bounded waits ran
 * out; *fault == 0 means none.  Synchronises `stream`. */
int mole_device_fault(void* stream, int32_t* fault);
/* the same check without a host wait, for a training loop: mole_device_fault_poll enqueues a copy
 * of the fault word (of the current device) into pinned host memory behind the work already on
 * `stream`; mole_device_fault_peek returns the value of the last such copy that has landed (0
 * before the first).  MOLECore polls at the end of every backward and peeks at the start of the
 * next forward.  On a stream that is being captured into a CUDA graph the poll does nothing
 * (its event would become part of the graph): poll behind a replay.  The reference has no
 * counterpart: its device code cannot time out. */
int mole_device_fault_poll(void* stream);
int mole_device_fault_peek(int32_t* fault);

/* kernels this library has launched in this process (the benchmark reports it) */
int mole_launch_count(int64_t* n);
/* while enabled every tensor-core grouped-GEMM launch is bracketed by CUDA events on its own
 * stream; mole_profile_read waits for them and returns the durations in launch order with
 * kind 0 = FC1, 1 = FC2, 2 = dX2, 3 = dX, 4 = weight gradient.  No counterpart in the
 * reference, which times whole phases (MOLE/utils/Utimer.py). */
int mole_profile_gemm(int32_t enable);
int mole_profile_read(float* ms, int32_t* kind, int32_t capacity, int32_t* n);

/* ------------------------------------------------------------------------------------
 * (a) gate + routing-index build.
 * Replaces MOLETopk.forward (MOLE/utils/Ugate.py:11-14) and the extract_critical call at
 * MOLE/moe/layer.py:445-447.
 * ---------------------------------------------------------------------------------- */
int mole_route_workspace_bytes(int64_t T, int32_t E, int32_t k, int64_t* bytes);

/* scores = softmax(x @ wg^T + logit_bias); top-k (ties to the lower expert id); slots by an
 * ordered scan (all j-th choices before any (j+1)-th, token order kept); kept iff slot < C.
 *   x [T,M] dtype, wg [E,M] dtype, logit_bias [E] f32 or NULL
 *   scores [T,E] f32, idx [T,k] i32, slot [T,k] i32, gates [T,k] f32 (0 where dropped)
 *   counts [E] i32 = min(hist, C), offsets [E+1] i32, perm [T*k] i32 (packed row -> t*k+j,
 *   -1 beyond offsets[E]), first_hist [E] i32 (first-choice histogram), l_aux [1] f32 */
int mole_gate_route_fwd(const void* x, const void* wg, const float* logit_bias,
                        int64_t T, int32_t M, int32_t E, int32_t k, int32_t C,
                        int32_t normalize_gate, int32_t dtype,
                        float* scores, int32_t* idx, int32_t* slot, float* gates,
                        int32_t* counts, int32_t* offsets, int32_t* perm,
                        int32_t* first_hist, float* l_aux,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* mole_gate_route_fwd for callers that cannot allocate a workspace.  Some hosts of this library
 * hand the whole of device memory to a pool of their own when they start (inference servers
 * that reserve HBM up front, trainers whose caching allocator is frozen after warm-up), or call
 * from a point where a driver allocation's implicit synchronisation would stall their other
 * streams; they can neither ask the driver for the routing scratch nor lend the library an
 * allocator.  This variant keeps the scratch in a fixed 4 MiB array inside the library's device
 * image, which every GPU that loads the library holds until the process exits.  It allocates
 * nothing (no cudaMalloc, no cudaFree, no allocating library routine).
 *   - limit: (k + 1) * ceil(T / 64) * E * 4 bytes <= 4 MiB (e.g. 32768 tokens, 128 experts,
 *     top-2, or 16384 tokens, 256 experts, top-3); larger problems get MOLE_ERR_UNSUPPORTED and
 *     must use mole_gate_route_fwd.
 *   - the first call on a device looks up the array's device address; make that call before
 *     any stream capture.
 *   - all calls share the one array and it keeps the last call's contents; nothing in it has to
 *     start at zero (each call writes every entry it later reads), but two calls whose kernels
 *     overlap on the GPU -- different streams, or different threads -- race on it.
 * No counterpart in the reference. */
int mole_gate_route_fwd_static(const void* x, const void* wg, const float* logit_bias,
                               int64_t T, int32_t M, int32_t E, int32_t k, int32_t C,
                               int32_t normalize_gate, int32_t dtype,
                               float* scores, int32_t* idx, int32_t* slot, float* gates,
                               int32_t* counts, int32_t* offsets, int32_t* perm,
                               int32_t* first_hist, float* l_aux, void* stream);

/* the same routing-index build from caller-provided scores [T,E] f32: identical scores in,
 * identical integers out */
int mole_route_from_scores(const float* scores, int64_t T, int32_t E, int32_t k, int32_t C,
                           int32_t normalize_gate,
                           int32_t* idx, int32_t* slot, float* gates,
                           int32_t* counts, int32_t* offsets, int32_t* perm,
                           int32_t* first_hist, float* l_aux,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* dlogits [T,E] f32 from the gradient of the gate weights dgates [T,k] (entries of dropped
 * pairs ignored) and of l_aux (d_l_aux [1] f32 device pointer or NULL) */
int mole_gate_bwd(const float* scores, const int32_t* idx, const int32_t* slot,
                  const float* dgates, const float* d_l_aux, const int32_t* first_hist,
                  int64_t T, int32_t E, int32_t k, int32_t C, int32_t normalize_gate,
                  float* dlogits, void* stream);

/* dwg32 [E,M] f32 += dlogits^T @ x   (caller zeroes dwg32 first when it wants "=").  The sum
 * over tokens is taken in two stages with a fixed order (per-chunk partial products in the
 * workspace, then one ordered reduction), so the result is bit-reproducible from run to run. */
int mole_gate_wgrad_workspace_bytes(int64_t T, int32_t M, int32_t E, int32_t dtype, int64_t* bytes);
int mole_gate_wgrad(const float* dlogits, const void* x, int64_t T, int32_t M, int32_t E,
                    int32_t dtype, float* dwg32, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* ------------------------------------------------------------------------------------
 * (b) dispatch / combine.  Replace fast_encode / fast_decode at
 * MOLE/moe/layer.py:448-449, 457-458 and their autograd.
 * ---------------------------------------------------------------------------------- */
/* disp[e*Cs + s] = x[t] for kept pairs; zero rows up to the next multiple of 128 */
int mole_dispatch_fwd(const void* x, const int32_t* counts, const int32_t* offsets,
                      const int32_t* perm, int64_t T, int32_t M, int32_t E, int32_t k,
                      int32_t Cs, int32_t dtype, void* disp, void* stream);
/* y[t] = sum_j gates[t,j] * rows[idx*Cs + slot]   (kept pairs) */
int mole_combine_fwd(const void* rows, const int32_t* idx, const int32_t* slot,
                     const float* gates, int64_t T, int32_t M, int32_t E, int32_t k,
                     int32_t C, int32_t Cs, int32_t dtype, void* y, void* stream);
/* backward of combine: drows[row] = gate * dy[t]; dgates[t,j] = <dy[t], rows[row]>;
 * pad rows of drows zeroed like dispatch */
int mole_combine_bwd(const void* dy, const void* rows, const float* gates,
                     const int32_t* counts, const int32_t* offsets, const int32_t* perm,
                     int64_t T, int32_t M, int32_t E, int32_t k, int32_t Cs, int32_t dtype,
                     void* drows, float* dgates, void* stream);

/* Push-style first exchange: dispatch (forward) and the combine's row gradient (backward) write
 * their valid rows straight into the receive buffer of each expert's owner.  peer_rows[q] is
 * rank q's buffer [W, L, Cs, M] mapped into this process, peer_counts[q] its int32 [W * L] count
 * array; row (e, s) of this rank lands in chunk (rank, e % L) of rank e / L.  No pad rows are
 * written: the receiver packs rows by count.  Replaces fast_encode + _BatchRecord::first_a2a
 * (MOLE/moe/layer.py:448-449, MOLE/cpp/core.cpp:144-179) and the backward mirror.
 *
 * Packed form (all_counts != NULL): all_counts is this rank's copy of every rank's counts,
 * int32 [W][E] (mole_peer_put_i32 + a barrier distribute it before the call).  The receive buffer
 * is then [L][W * Cs][M], one run per local expert, and the sender puts its rows straight at
 * their final place in the run, behind the rows of the lower ranks: the receiver has nothing to
 * gather (mole_ffn_*_peer with desc.compact = 3).  peer_counts is not used in this form. */
int mole_dispatch_fwd_peer(const void* x, const int32_t* counts, const int32_t* offsets,
                           const int32_t* perm, int64_t T, int32_t M, int32_t E, int32_t k,
                           int32_t Cs, int32_t dtype, void* const* peer_rows,
                           int32_t* const* peer_counts, const int32_t* all_counts,
                           int32_t n_peers, int32_t rank, void* stream);
int mole_combine_bwd_peer(const void* dy, const void* rows, const float* gates,
                          const int32_t* counts, const int32_t* offsets, const int32_t* perm,
                          int64_t T, int32_t M, int32_t E, int32_t k, int32_t Cs, int32_t dtype,
                          void* const* peer_rows, const int32_t* all_counts, int32_t n_peers,
                          int32_t rank, float* dgates, void* stream);
/* src[0..n) of this rank into slot `rank` of every rank's int32 [world][n] table (peer_tables[q]
 * = rank q's table mapped into this process, this rank's own for q == rank).  Used to tell every
 * rank every rank's per-expert row counts; follow it with a barrier before reading the table. */
int mole_peer_put_i32(const int32_t* src, int32_t n, void* const* peer_tables, int32_t world,
                      int32_t rank, void* stream);
/* backward of dispatch fused with the gate's input gradient:
 * dx[t] = sum_j kept * ddisp[idx*Cs + slot] + dlogits[t,:] @ wg
 * (ddisp may be NULL: gate term only; dlogits and wg may both be NULL: dispatch term only) */
int mole_dispatch_bwd(const void* ddisp, const int32_t* idx, const int32_t* slot,
                      const float* dlogits, const void* wg,
                      int64_t T, int32_t M, int32_t E, int32_t k, int32_t C, int32_t Cs,
                      int32_t dtype, void* dx, void* stream);

/* ------------------------------------------------------------------------------------
 * (c) grouped expert FFN.  Replaces _BatchRecord::bffn_fwd / bffn_bwd / bffn_bwd_acc
 * (MOLE/cpp/core.cpp:344-367, 381-456, 457-514), the re-layouts either side of them
 * (core.cpp:233, 240, 291, 320) and the GELU' kernel (MOLE/cpp/gelu.cu:16-58).
 *
 * The workspace is scratch of one call (tile schedule; with n_src > 1 on the tensor-core path
 * also the packed copies of x and dout and the row map).  x1, h and dx1 are private to the
 * fwd/bwd pair: backward must be called with the descriptor fields n_src, Cs, L, dtype, backend,
 * compact that forward used.
 * Rows are capacity-strided: chunk c = w*L + l holds what source rank w sent for local
 * expert l (n_src = 1 on a single GPU).  counts [n_src*L] i32 lives on the device; no
 * host synchronisation happens.  Weights are batched [n_slots, F, M] (W1 and W2 both, as in
 * MOLE/moe/layer.py:89-96), biases [n_slots, F] / [n_slots, M]; expert l uses slot
 * slot_of_expert[l] (host array, NULL = identity).  Only experts [e_begin, e_end) are
 * processed, which is how the offload pipeline runs the layer one expert batch at a time.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  int32_t dtype;          /* mole_dtype */
  int32_t act;            /* mole_act */
  int32_t gelu_bwd;       /* mole_gelu_bwd */
  int32_t M, F;           /* embed dim, ffn dim */
  int32_t L;              /* local experts */
  int32_t n_src;          /* source ranks (chunks per local expert) */
  int32_t Cs;             /* chunk stride in rows, multiple of 128 */
  int32_t e_begin, e_end; /* local expert range to process */
  int32_t n_slots;        /* leading extent of the weight arrays */
  int32_t n_grad_slots;   /* leading extent of the gradient arrays (0: same as n_slots) */
  int32_t accumulate;     /* backward: weight grads += instead of = (core.cpp:457-514) */
  int32_t compact;        /* 0: with n_src > 1 the tensor-core path packs each expert's rows of all
                             sources into one run before the GEMMs (x1, h, dx1 are then in that
                             layout); 2: never pack; 3: x and dout already ARE packed,
                             [L][n_src * Cs][M] with expert l's rows of all sources in source order
                             at the front of its run (the packed form of mole_dispatch_fwd_peer /
                             mole_combine_bwd_peer): nothing is gathered, the call writes the pad
                             rows of x (forward) and dout (backward) in place */
  int32_t backend;        /* 0: tensor cores for bf16, CUDA cores for fp32 (the fp32 layer needs
                             fp32-exact products).  For bf16, 0 picks per launch: the panel kernel
                             (weights on the M side of the MMA, an expert's rows on N) for row
                             GEMMs up to 1024 rows per expert whose rows are one run and whose
                             outputs stay in place, the resident-operand kernel for weight
                             gradients of experts with at most 512 rows, otherwise 128x256 tiles
                             (one CTA) or 256x256 tiles (CTA pairs) by the number of row tiles an
                             expert can have.
                             1: CUDA-core kernels also for bf16, used to bisect numerics;
                             2: the one-CTA tile kernel everywhere; 3: CTA-pair tile kernels
                             wherever the shape allows; 4: panel and resident-operand kernels
                             wherever they are eligible (2-4 exist for A/B comparisons; all
                             tensor-core back ends give bit-identical rows and weight
                             gradients; gb1 comes out of the panel kernel's dX2 epilogue where that
                             kernel runs -- the same values added in another fixed order) */
} mole_ffn_desc;

/* scratch the FFN needs per call (tile schedule, packed-row map, partial column sums of the
 * panel kernel); bytes depends only on dtype, backend, compact, L, n_src, Cs, M and F */
int mole_ffn_workspace_bytes(const mole_ffn_desc* d, int64_t* bytes);

/* x rows [n_src*L*Cs, M] -> out rows [.., M]; saves pre-activation x1 and activation h
 * (both [.., F]) for backward */
int mole_ffn_fwd(const mole_ffn_desc* d, const int32_t* counts, const int32_t* slot_of_expert,
                 const void* x, const void* w1, const void* b1, const void* w2, const void* b2,
                 void* x1, void* h, void* out,
                 void* workspace, int64_t workspace_bytes, void* stream);

/* mole_ffn_fwd with the gate-weighted combine (fast_decode, MOLE/moe/layer.py:456-458) fused into
 * the second GEMM's epilogue: besides storing out, FC2 adds gates[pair] * out[row] into
 * y[token] ([T, M], zeroed by the caller) for every valid row, row (e, s) being pair
 * perm[offsets[e] + s] = token * k + choice (the arrays of mole_gate_route_fwd).  bf16, one
 * source rank, k <= 2 (two addends commute: the result does not depend on the order in which
 * the reductions land); other cases get MOLE_ERR_UNSUPPORTED and use mole_combine_fwd. */
int mole_ffn_fwd_combine(const mole_ffn_desc* d, const int32_t* counts,
                         const int32_t* slot_of_expert, const void* x, const void* w1,
                         const void* b1, const void* w2, const void* b2, void* x1, void* h,
                         void* out, const int32_t* offsets, const int32_t* perm,
                         const float* gates, int32_t k, void* y,
                         void* workspace, int64_t workspace_bytes, void* stream);

/* dout rows -> dx rows (NULL to skip) and weight grads gw1,gw2 [n_slots,F,M], gb1 [n_slots,F],
 * gb2 [n_slots,M].  dx1 [.., F] is caller-provided scratch. */
int mole_ffn_bwd(const mole_ffn_desc* d, const int32_t* counts, const int32_t* slot_of_expert,
                 const int32_t* grad_slot_of_expert,
                 const void* dout, const void* x, const void* x1, const void* h,
                 const void* w1, const void* w2,
                 void* dx1, void* dx, void* gw1, void* gb1, void* gw2, void* gb2,
                 void* workspace, int64_t workspace_bytes, void* stream);

/* The same two calls with the return exchange fused into the last GEMM: the output rows (FC2 in
 * forward, dX in backward) are stored straight into the source ranks' receive buffers instead of
 * a local buffer that an all-to-all then sends.  peer_out[w] / peer_dx[w] is rank w's buffer
 * [E_total, Cs, M] mapped into this process (mole_peer_open; this rank's own buffer for
 * w == rank); the rows of chunk (w, l) land in chunk rank * L + l of it.  bf16 tensor-core path
 * with n_src > 1 only.  Replaces _BatchRecord::second_a2a (MOLE/cpp/core.cpp:180-210) and its
 * backward mirror; the caller orders readers behind the writers with mole_barrier. */
int mole_ffn_fwd_peer(const mole_ffn_desc* desc, const int32_t* counts,
                      const int32_t* slot_of_expert, const void* x, const void* w1, const void* b1,
                      const void* w2, const void* b2, void* x1, void* h, void* const* peer_out,
                      int32_t rank, void* workspace, int64_t workspace_bytes, void* stream);
int mole_ffn_bwd_peer(const mole_ffn_desc* desc, const int32_t* counts,
                      const int32_t* slot_of_expert, const int32_t* grad_slot_of_expert,
                      const void* dout, const void* x, const void* x1, const void* h,
                      const void* w1, const void* w2, void* dx1, void* const* peer_dx,
                      int32_t rank, void* gw1, void* gb1, void* gw2, void* gb2, void* workspace,
                      int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------
 * streams.  Replaces the 16-stream manager (MOLE/cpp/stream.cpp:38-144) and its wait
 * helpers (stream.cpp:156-205).  Roles follow the reference: 1 = H2D transfer, 2 = compute,
 * 3 = communication, 4 = D2H transfer.
 * ---------------------------------------------------------------------------------- */
typedef struct mole_ctx mole_ctx;
int mole_ctx_create(int32_t device, int32_t single_stream, mole_ctx** ctx);
int mole_ctx_destroy(mole_ctx* ctx);
/* cudaStream_t of role `idx` in [0,16) for interop (torch.cuda.ExternalStream) */
int mole_ctx_stream(mole_ctx* ctx, int32_t idx, void** stream);
/* make stream `waiter` wait for everything enqueued so far on stream `waited` */
int mole_ctx_wait(mole_ctx* ctx, void* waiter, void* waited);
/* per-record edges (comp_event / comm_event / para_event of MOLE/cpp/define.hpp:634-636):
 * record returns a ticket for the work enqueued on `stream` so far; wait orders `stream` behind
 * that work only.  The last 1024 tickets stay valid. */
int mole_ctx_event_record(mole_ctx* ctx, void* stream, int64_t* ticket);
int mole_ctx_event_wait(mole_ctx* ctx, int64_t ticket, void* stream);
int mole_ctx_synchronize(mole_ctx* ctx, int32_t idx);

/* ------------------------------------------------------------------------------------
 * (d) expert-parallel exchange.  Replaces ensure_nccl / MOLEAll2Allfp32
 * (MOLE/cpp/communication.cpp:49-100).
 * ---------------------------------------------------------------------------------- */
typedef struct mole_comm mole_comm;
/* writes a 128-byte NCCL unique id (rank 0 calls this, then broadcasts the bytes) */
int mole_comm_unique_id(uint8_t* id128);
int mole_comm_create(const uint8_t* id128, int32_t world_size, int32_t rank, int32_t device,
                     mole_comm** comm);
int mole_comm_destroy(mole_comm* comm);
/* equal-split all-to-all of bytes: bytes_per_peer bytes at send + q*peer_stride_bytes go to
 * rank q and land at recv + r*peer_stride_bytes on it (r = sender); the self chunk is a device
 * copy.  Grouped ncclSend/ncclRecv on `stream`.  A stride larger than the payload exchanges one
 * expert batch of a capacity-strided buffer (MOLE/cpp/core.cpp:156-161) without re-layout. */
int mole_all2all(mole_comm* comm, const void* send, void* recv, int64_t bytes_per_peer,
                 int64_t peer_stride_bytes, void* stream);

/* Peer-visible device buffers for the push-style exchange: the owner allocates (plain device
 * memory, zeroed) and exports a 64-byte CUDA IPC handle; a peer process opens it and passes the
 * mapped pointer to the *_peer entry points, whose kernels store rows straight into it over
 * NVLink (replaces the send buffer + grouped ncclSend/ncclRecv of MOLE/cpp/core.cpp:144-210,
 * MOLE/cpp/communication.cpp:68-100).  mole_barrier: every rank has finished what it enqueued
 * on `stream` before the call (4-byte grouped send/recv with every peer); `scratch` is 8 * world
 * bytes of device memory. */
int mole_peer_alloc(int64_t bytes, void** ptr);
int mole_peer_free(void* ptr);
int mole_peer_export(void* ptr, uint8_t* handle64);
int mole_peer_open(const uint8_t* handle64, void** ptr);
int mole_peer_close(void* ptr);
int mole_barrier(mole_comm* comm, void* scratch, void* stream);
/* the same barrier through flags in peer-visible memory instead of NCCL: peer_flags[q] is rank q's
 * int32 [world] array (mole_peer_alloc'ed, zeroed) mapped into this process; `seq` is the
 * barrier's sequence number, 1, 2, 3, ... identical on every rank.  One tiny kernel stores seq
 * into entry `rank` of every peer's array and waits, at most limit_ns, until its own array shows
 * seq (or more) from every peer; when the wait runs out it records 40 + the missing rank in the
 * device fault word (mole_device_fault) and returns -- nothing hangs. */
int mole_peer_barrier(void* const* peer_flags, int32_t world, int32_t rank, int32_t seq,
                      int64_t limit_ns, void* stream);

/* ------------------------------------------------------------------------------------
 * (e) offloaded experts.  Replaces _UniMem (MOLE/cpp/define.hpp:143-193,
 * MOLE/cpp/umemory.cpp:92-205), _CPUParamCore::prefetch_to / store_batch_grad
 * (MOLE/cpp/uparameter.cpp:58-71) and the copy wrappers (MOLE/cpp/transfer.cu:4-21).
 * The pool owns pool_size expert slots for each of the four parameter kinds
 * (W1 [F,M], b1 [F], W2 [F,M], b2 [M]); this is the one place the library allocates
 * device memory, once, at creation.
 * ---------------------------------------------------------------------------------- */
typedef struct mole_pool mole_pool;
/* ctx == NULL creates a pool without device memory that only records what it would do
 * (mole_pool_log); the slot / prefetch-stack logic is identical */
int mole_pool_create(mole_ctx* ctx, int32_t pool_size, int32_t M, int32_t F, int32_t dtype,
                     mole_pool** pool);
int mole_pool_destroy(mole_pool* pool);
/* device base pointer of parameter kind p_id in [0,4): [pool_size, ...] */
int mole_pool_base(mole_pool* pool, int32_t p_id, void** base);
/* slots currently visible to forward/backward (pool_size minus prefetch reservations) */
int mole_pool_view_size(mole_pool* pool, int32_t* n);
int mole_pool_clear_virtual(mole_pool* pool);
/* reserve the next n slots for layer moe_id, push (moe_id, n) on the prefetch stack and
 * return the first reserved slot (umemory.cpp:131-154) */
int mole_pool_prefetch(mole_pool* pool, int32_t moe_id, int32_t n, int32_t* first_slot);
/* pop the reservation of layer moe_id if it is on top of the stack; *n = 0 otherwise
 * (umemory.cpp:169-183) */
int mole_pool_pop_prefetched(mole_pool* pool, int32_t moe_id, int32_t* n);
/* H2D copy of experts [e0, e0+n) of the four pinned host arrays into view slots
 * [slot0, slot0+n) (absolute slots when `absolute` != 0, as a prefetch into slots it has just
 * reserved needs) on the transfer stream, skipping the first `skip` experts (already
 * prefetched).  Waits for the compute that last used those slots; records the fetch so that
 * mole_pool_wait_fetch can order the compute stream after it. */
int mole_pool_fetch(mole_pool* pool, const void* const host_params[4], int64_t e0, int32_t n,
                    int32_t slot0, int32_t skip, int32_t absolute, int32_t* ticket);
int mole_pool_wait_fetch(mole_pool* pool, int32_t ticket, void* stream);
/* tell the pool that work enqueued on `stream` so far is the last user of view slots
 * [slot0, slot0+n): a later fetch into them waits for it */
int mole_pool_mark_used(mole_pool* pool, int32_t slot0, int32_t n, void* stream);
/* recorded plan of a ctx == NULL pool: entries {kind, a, b, c} with kind 0 = copy of c experts
 * from expert a into absolute slot b, 1 = slots [a, a+b) marked used, 2 = copy waits for the
 * last user of slot a */
int mole_pool_log(mole_pool* pool, int32_t* out, int32_t capacity, int32_t* n_entries);
/* absolute slot index of view slot s (adds the prefetch offset) */
int mole_pool_abs_slot(mole_pool* pool, int32_t view_slot, int32_t* abs_slot);
/* D2H copy of `bytes` from device to pinned host on the D2H stream after `after_stream`'s
 * current work */
int mole_store_to_host(mole_ctx* ctx, void* host_dst, const void* dev_src, int64_t bytes,
                       void* after_stream);

/* ------------------------------------------------------------------------------------
 * optimizer step of offloaded experts on the GPU ("instant Adam") and the cross-layer prefetch
 * assignment.  Replace _MOLECore::adam / instant_adam (MOLE/cpp/define.hpp:543-579,
 * MOLE/cpp/core.cpp:848-943) and _fast_assign_prefetch (MOLE/cpp/core.cpp:1302-1345).
 * ---------------------------------------------------------------------------------- */
/* One fused pass over n elements, in place: p, m, v updated from g (+ g_extra when not NULL: a
 * gradient accumulated over earlier micro-steps).  t is the step count AFTER this step (the
 * reference's this->t + 1).  adamw != 0: decoupled weight decay p *= 1 - lam*lr; else g += lam*p.
 * All five arrays have element type `dtype`; the arithmetic is fp32. */
int mole_adam_update(void* p, void* m, void* v, const void* g, const void* g_extra, int64_t n,
                     int32_t dtype, float beta1, float beta2, int32_t t, float lr, float lam,
                     float eps, int32_t adamw, void* stream);
/* P free pool slots, n layers, layer i can hide F[i] expert fetches and owns E[i] offloaded
 * experts.  local[i] = experts layer i prefetches for itself; triples[3j..3j+2] = (lender layer,
 * borrower layer, count): while the lender runs it also fetches `count` experts of the borrower.
 * Host-only (no device work).  *n_triples is the number found even when it exceeds capacity. */
int mole_fast_assign_prefetch(int32_t P, const int32_t* F, const int32_t* E, int32_t n,
                              int32_t* local, int32_t* triples, int32_t capacity,
                              int32_t* n_triples);

#ifdef __cplusplus
}
#endif
#endif /* MOLE_B200_H_ */
