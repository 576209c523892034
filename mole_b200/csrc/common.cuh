// Shared helpers for the mole_b200 CUDA library: status handling, element-type traits and
// the activation math used by both grouped-GEMM back ends.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/mole_b200.h"

namespace mole {

// ---- error reporting --------------------------------------------------------------
char* last_error_buffer();   // thread-local, 512 bytes
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define MOLE_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::mole::fail(MOLE_ERR_CUDA, "%s:%d %s -> %s", __FILE__, __LINE__, #expr,   \
                          cudaGetErrorString(_e));                                      \
  } while (0)

#define MOLE_REQUIRE(cond, ...)                                       \
  do {                                                                \
    if (!(cond)) return ::mole::fail(MOLE_ERR_INVALID, __VA_ARGS__);  \
  } while (0)

// after every kernel launch: counts it (mole_launch_count) and surfaces launch errors
void count_launch();
#define MOLE_LAUNCH_OK()          \
  do {                            \
    ::mole::count_launch();       \
    MOLE_CUDA_OK(cudaGetLastError()); \
  } while (0)

// optional per-launch timing of the grouped GEMMs (mole_profile_gemm / mole_profile_read)
bool profile_enabled();
void profile_begin(cudaStream_t st, int kind);
void profile_end(cudaStream_t st);

// bf16 backward products of the gate on warp-level tensor cores (gate_mma.cu); need M % 128 == 0
int launch_dispatch_bwd_mma(const void* ddisp, const int32_t* idx, const int32_t* slot,
                            const float* dlogits, const void* wg, int64_t T, int M, int E, int k,
                            int C, int Cs, void* dx, cudaStream_t st);
int launch_gate_wgrad_mma(const float* dlogits, const void* x, int64_t T, int M, int E, int chunk,
                          int n_chunks, float* partial, cudaStream_t st);

// device-side fault word: kernels with bounded waits record where they gave up
int32_t* device_fault_word();   // of the current device; allocated at its first use (256 bytes), zeroed

// Per-device host state.  cudaFuncSetAttribute, occupancy figures and the SM count belong to a
// device, not to the process: a process that drives several GPUs needs them once per device.
constexpr int kMaxDevices = 64;
inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}
// One int per device, 0 until set.  Racing setters write the same value, so plain atomics do.
struct PerDeviceInt {
  std::atomic<int64_t> v[kMaxDevices];
  int64_t get(int dev) const { return v[dev].load(std::memory_order_acquire); }
  void set(int dev, int64_t x) { v[dev].store(x, std::memory_order_release); }
};
int sm_count();                 // multiprocessors of the current device

// ---- element types ---------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;   // elements per 16-byte vector
  __device__ static __forceinline__ float to_f(float v) { return v; }
  __device__ static __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector load/store of T converted to/from float registers
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---- activation math ----------------------------------------------------------------
__device__ __forceinline__ float gelu_exact(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}
__device__ __forceinline__ float gelu_exact_grad(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
  const float pdf = 0.39894228040143267794f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
// derivative of the tanh approximation, as the reference's own kernel computes it
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float c = 0.7978845608028654f, a = 0.044715f;
  const float t = tanhf(c * (x + a * x * x * x));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * c * (1.0f + 3.0f * a * x * x);
}
__device__ __forceinline__ float act_fwd(float x, int act) {
  return act == MOLE_ACT_GELU ? gelu_exact(x) : fmaxf(x, 0.0f);
}
__device__ __forceinline__ float act_grad(float x, int act, int gelu_bwd) {
  if (act == MOLE_ACT_RELU) return x > 0.0f ? 1.0f : 0.0f;
  return gelu_bwd == MOLE_GELU_BWD_TANH ? gelu_tanh_grad(x) : gelu_exact_grad(x);
}

// ---- grouped GEMM plumbing shared by the two back ends ------------------------------
// Tile schedule built on the device from the per-chunk row counts (no host sync):
//   tile_row0[i]   first row of the i-th 128-row tile that holds at least one valid row
//   tile_expert[i] local expert the tile belongs to; tiles are sorted by expert
//   expert_tile_start[l - e_begin] .. [+1]  tile index range of expert l
//   expert_pair_start  the same ranges counted in pairs of tiles (odd counts rounded up)
//   n_tiles        total
// Push-style exchange: where row (e, s) of a rank's expert-major [E][Cs] row space lives when it
// is written straight into the memory of the expert's owner.  Rank q owns experts
// [q * L, (q + 1) * L); its receive buffer is [W][L][Cs][width] (chunk [w][l] = what rank w
// sent for local expert l) and base[q] is that buffer mapped into this process.
constexpr int kMaxPeers = 16;
struct PeerMap {
  void* base[kMaxPeers];
  int32_t* counts[kMaxPeers];     // rank q's [W * L] valid-row counts (dispatch only), or null
  int n;                          // ranks; 0: no peers, rows stay local
  int rank, L;
  // Packed layout: when every rank knows every rank's counts ([W][E] table, local copy here), a
  // sender puts its rows straight at their final place in the owner's per-expert run
  // [L][W * Cs]: behind the rows of the lower ranks.  Null: chunk layout [W][L][Cs].
  const int32_t* all_counts;
  int E;
};
// Order in which a pushing kernel walks the experts: rank r starts with the experts of rank r + 1
// and ends with its own.  In natural order every rank would store to rank 0's memory first, then
// to rank 1's ...: all senders on one receiver's links at a time.  Rotated, the ranks' targets
// are a permutation at every moment.
__device__ __forceinline__ int peer_rotate_expert(const PeerMap& pm, int e) {
  const int shifted = e + ((pm.rank + 1) % pm.n) * pm.L;
  return shifted >= pm.E ? shifted - pm.E : shifted;
}
__device__ __forceinline__ int64_t peer_row(const PeerMap& pm, int e, int s, int Cs, int* owner) {
  *owner = e / pm.L;
  const int l = e - *owner * pm.L;
  if (pm.all_counts != nullptr) {
    int base = 0;
    for (int w = 0; w < pm.rank; ++w) base += min(pm.all_counts[w * pm.E + e], Cs);
    return (int64_t)l * pm.n * Cs + base + s;
  }
  return ((int64_t)pm.rank * pm.L + l) * Cs + s;
}

struct Schedule {
  int32_t* n_tiles;            // [1]
  int32_t* expert_tile_start;  // [L + 1]
  int32_t* expert_pair_start;  // [L + 1]  prefix of ceil(tiles / 2): work units of the 2-CTA GEMM
  int32_t* tile_row0;          // [max_tiles]
  int32_t* tile_expert;        // [max_tiles]
  int32_t* tile_rows;          // [max_tiles]  valid rows of the tile (1..128); the rest are zero rows
  int32_t max_tiles;
};

enum Epilogue : int {
  EPI_FC1 = 0,     // v = acc + bias[n]; out0 = v (pre-activation); out1 = act(v)
  EPI_BIAS = 1,    // out0 = acc + bias[n]
  EPI_DACT = 2,    // out0 = acc * act'(aux[row, n])
  EPI_STORE = 3,   // out0 = acc
  EPI_WGRAD = 4    // per-expert output [F, M]: out0[slot] (+)= acc
};

constexpr int kTileRows = 128;

}  // namespace mole
