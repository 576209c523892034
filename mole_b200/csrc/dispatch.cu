// (b) Dispatch / combine over capacity-strided rows, forward and backward.
//
// Replaces the fast_encode / fast_decode calls at MOLE/moe/layer.py:448-449, 457-458 and
// their autograd.  All four kernels move whole rows with 16-byte vectors; a warp owns a row
// (or a token) and keeps several vectors in flight per lane.  They are HBM-bound:
//   dispatch_fwd   reads P rows, writes P rows (+ zero pad rows)            2*P*M*s bytes
//   combine_fwd    reads P rows, writes T rows                              (P+T)*M*s
//   combine_bwd    reads P rows of dy (L2 hits for the 2nd choice) + P rows of expert output,
//                  writes P rows                                            3*P*M*s
//   dispatch_bwd   reads P rows, writes T rows (+ the tiny dlogits @ Wg)    (P+T)*M*s
#include "common.cuh"

namespace mole {

constexpr int kRowWarps = 8;   // rows (or tokens) per 256-thread block

// Row-driven: one warp per destination row of the [E][Cs] buffer.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
dispatch_fwd_kernel(const T* __restrict__ x, const int32_t* __restrict__ counts,
                    const int32_t* __restrict__ offsets, const int32_t* __restrict__ perm,
                    int M, int E, int k, int Cs, T* __restrict__ disp,
                    const __grid_constant__ PeerMap pm) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (row >= (int64_t)E * Cs) return;
  const int e_walk = (int)(row / Cs), s = (int)(row - (int64_t)e_walk * Cs);
  const int e = pm.n > 0 ? peer_rotate_expert(pm, e_walk) : e_walk;
  const int cnt = counts[e];
  uint4* dst;
  if (pm.n > 0) {
    // pushed to the expert's owner: valid rows only (the receiver packs rows by count and pads
    // there), and the count itself
    int owner;
    const int64_t prow = peer_row(pm, e, s, Cs, &owner);
    if (pm.all_counts == nullptr && s == 0 && lane == 0) pm.counts[owner][prow / Cs] = cnt;
    if (s >= cnt) return;
    dst = reinterpret_cast<uint4*>(static_cast<T*>(pm.base[owner]) + prow * M);
  } else {
    dst = reinterpret_cast<uint4*>(disp + row * M);       // e == e_walk here
  }
  const int padded = (cnt + kTileRows - 1) / kTileRows * kTileRows;
  if (s >= padded) return;
  const int nvec = M / V;
  if (s >= cnt) {
    for (int i = lane; i < nvec; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int pair = perm[offsets[e] + s];
  const int64_t t = pair / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + t * M);
  int i = lane;
  for (; i + 96 < nvec; i += 128) {
    const uint4 a = __ldg(src + i), b = __ldg(src + i + 32), c = __ldg(src + i + 64),
                d = __ldg(src + i + 96);
    dst[i] = a; dst[i + 32] = b; dst[i + 64] = c; dst[i + 96] = d;
  }
  for (; i < nvec; i += 32) dst[i] = __ldg(src + i);
}

// Token-driven: one warp per token, fp32 accumulation over its k rows.  The token's (row, gate)
// pairs are read once; for k <= 2 the loop over the row's vectors keeps four vectors per source
// row in flight per lane (eight 16-byte loads): with one vector per source row in flight the
// kernel reached 0.68 of the copy bandwidth.
template <typename T, int K>
__device__ __forceinline__ void combine_token(const T* __restrict__ rows, const int64_t (&r)[K],
                                              const float (&g)[K], int nvec, int M, int lane,
                                              T* __restrict__ yrow) {
  constexpr int V = Vec16<T>::N;
  constexpr int U = 4;
  int i = lane;
  for (; i + 32 * (U - 1) < nvec; i += 32 * U) {
    float v[K][U][V];
#pragma unroll
    for (int j = 0; j < K; ++j)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (r[j] >= 0) {
          Vec16<T>::load(rows + r[j] * M + (int64_t)(i + 32 * u) * V, v[j][u]);
        } else {
#pragma unroll
          for (int c = 0; c < V; ++c) v[j][u][c] = 0.f;
        }
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float acc[V];
#pragma unroll
      for (int c = 0; c < V; ++c) acc[c] = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j)
#pragma unroll
        for (int c = 0; c < V; ++c) acc[c] = fmaf(g[j], v[j][u][c], acc[c]);
      Vec16<T>::store(yrow + (int64_t)(i + 32 * u) * V, acc);
    }
  }
  for (; i < nvec; i += 32) {
    float acc[V];
#pragma unroll
    for (int c = 0; c < V; ++c) acc[c] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (r[j] < 0) continue;
      float v[V];
      Vec16<T>::load(rows + r[j] * M + (int64_t)i * V, v);
#pragma unroll
      for (int c = 0; c < V; ++c) acc[c] = fmaf(g[j], v[c], acc[c]);
    }
    Vec16<T>::store(yrow + (int64_t)i * V, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_fwd_kernel(const T* __restrict__ rows, const int32_t* __restrict__ idx,
                   const int32_t* __restrict__ slot, const float* __restrict__ gates,
                   int64_t Ttok, int M, int k, int C, int Cs, T* __restrict__ y) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (t >= Ttok) return;
  const int nvec = M / V;
  if (k <= 2) {
    int64_t r[2];
    float g[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      r[j] = -1;
      g[j] = 0.f;
      if (j < k) {
        const int s = slot[t * k + j];
        if (s < C) {
          r[j] = (int64_t)idx[t * k + j] * Cs + s;
          g[j] = gates[t * k + j];
        }
      }
    }
    combine_token<T, 2>(rows, r, g, nvec, M, lane, y + t * M);
    return;
  }
  for (int i = lane; i < nvec; i += 32) {
    float acc[V];
#pragma unroll
    for (int c = 0; c < V; ++c) acc[c] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int s = slot[t * k + j];
      if (s >= C) continue;
      const float g = gates[t * k + j];
      const int64_t r = (int64_t)idx[t * k + j] * Cs + s;
      float v[V];
      Vec16<T>::load(rows + r * M + (int64_t)i * V, v);
#pragma unroll
      for (int c = 0; c < V; ++c) acc[c] = fmaf(g, v[c], acc[c]);
    }
    Vec16<T>::store(y + t * M + (int64_t)i * V, acc);
  }
}

// Row-driven: drows[row] = g * dy[t];  dgates[pair] = <dy[t], rows[row]>.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ rows,
                   const float* __restrict__ gates, const int32_t* __restrict__ counts,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ perm, int M,
                   int E, int k, int Cs, T* __restrict__ drows, float* __restrict__ dgates,
                   const __grid_constant__ PeerMap pm) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (row >= (int64_t)E * Cs) return;
  const int e_walk = (int)(row / Cs), s = (int)(row - (int64_t)e_walk * Cs);
  const int e = pm.n > 0 ? peer_rotate_expert(pm, e_walk) : e_walk;
  const int cnt = counts[e];
  const int padded = (cnt + kTileRows - 1) / kTileRows * kTileRows;
  if (s >= padded) return;
  const int nvec = M / V;
  T* dst;
  if (pm.n > 0) {                      // gradient rows go straight to the expert's owner
    if (s >= cnt) return;
    int owner;
    const int64_t prow = peer_row(pm, e, s, Cs, &owner);
    dst = static_cast<T*>(pm.base[owner]) + prow * M;
  } else {
    dst = drows + row * M;
  }
  if (s >= cnt) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = lane; i < nvec; i += 32) d4[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int pair = perm[offsets[e] + s];
  const int64_t t = pair / k;
  const float g = gates[pair];
  const T* dyr = dy + t * M;
  const T* orow = rows + ((int64_t)e * Cs + s) * M;      // the expert's row, not the walk position
  float dot = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float a[V], b[V], o[V];
    Vec16<T>::load(dyr + (int64_t)i * V, a);
    Vec16<T>::load(orow + (int64_t)i * V, b);
#pragma unroll
    for (int c = 0; c < V; ++c) {
      dot = fmaf(a[c], b[c], dot);
      o[c] = g * a[c];
    }
    Vec16<T>::store(dst + (int64_t)i * V, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dgates[pair] = dot;
}

// dx[t, :] = sum_j kept * ddisp[row(t, j), :] + dlogits[t, :] @ Wg.
// Block: 32 tokens x 128 columns; the gate term is a small register-tiled product over E.
constexpr int kDbTok = 32, kDbCols = 128, kDbEC = 32;
template <typename T>
__global__ void __launch_bounds__(256)
dispatch_bwd_kernel(const T* __restrict__ ddisp, const int32_t* __restrict__ idx,
                    const int32_t* __restrict__ slot, const float* __restrict__ dlogits,
                    const T* __restrict__ wg, int64_t Ttok, int M, int E, int k, int C, int Cs,
                    T* __restrict__ dx) {
  __shared__ float dl_s[kDbTok][kDbEC + 1];
  __shared__ float wg_s[kDbEC][kDbCols + 4];
  const int tid = threadIdx.x;
  const int tg = tid >> 5, cg = tid & 31;          // token group (4 tokens), column group (4 cols)
  const int64_t tok0 = (int64_t)blockIdx.y * kDbTok;
  const int col0 = blockIdx.x * kDbCols;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
  if (dlogits != nullptr) {
    for (int e0 = 0; e0 < E; e0 += kDbEC) {
      for (int i = tid; i < kDbTok * kDbEC; i += 256) {
        const int tl = i / kDbEC, e = i - tl * kDbEC;
        const int64_t t = tok0 + tl;
        dl_s[tl][e] = (t < Ttok && e0 + e < E) ? dlogits[t * E + e0 + e] : 0.f;
      }
      for (int i = tid; i < kDbEC * kDbCols; i += 256) {
        const int e = i / kDbCols, c = i - e * kDbCols;
        wg_s[e][c] = (e0 + e < E && col0 + c < M)
                         ? Elem<T>::to_f(wg[(int64_t)(e0 + e) * M + col0 + c]) : 0.f;
      }
      __syncthreads();
#pragma unroll 8
      for (int e = 0; e < kDbEC; ++e) {
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = dl_s[tg * 4 + i][e];
        const float4 b = *reinterpret_cast<const float4*>(&wg_s[e][cg * 4]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
          acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
          acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
          acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
        }
      }
      __syncthreads();
    }
  }
  const int col = col0 + cg * 4;
  if (col >= M) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t t = tok0 + tg * 4 + i;
    if (t >= Ttok) continue;
    for (int j = 0; j < k && ddisp != nullptr; ++j) {
      const int s = slot[t * k + j];
      if (s >= C) continue;
      const int64_t r = (int64_t)idx[t * k + j] * Cs + s;
      const T* p = ddisp + r * M + col;
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][c] += Elem<T>::to_f(p[c]);
    }
    T* o = dx + t * M + col;
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] = Elem<T>::from_f(acc[i][c]);
  }
}

static int check_rows(int64_t T, int M, int E, int k, int Cs, int dtype) {
  MOLE_REQUIRE(T > 0 && E > 0 && k > 0, "bad sizes T=%lld E=%d k=%d", (long long)T, E, k);
  MOLE_REQUIRE(Cs > 0 && Cs % kTileRows == 0, "Cs=%d must be a positive multiple of %d", Cs, kTileRows);
  const int vec = dtype == MOLE_F32 ? 4 : 8;
  MOLE_REQUIRE(dtype == MOLE_F32 || dtype == MOLE_BF16, "dtype %d", dtype);
  MOLE_REQUIRE(M > 0 && M % vec == 0, "M=%d must be a multiple of %d (16-byte rows)", M, vec);
  return MOLE_OK;
}

}  // namespace mole

using namespace mole;

#define MOLE_BY_DTYPE(dtype, ...)                                     \
  if ((dtype) == MOLE_F32) { using T = float; __VA_ARGS__; }          \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

extern "C" int mole_dispatch_fwd(const void* x, const int32_t* counts, const int32_t* offsets,
                                 const int32_t* perm, int64_t T_, int32_t M, int32_t E, int32_t k,
                                 int32_t Cs, int32_t dtype, void* disp, void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(x && counts && offsets && perm && disp, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(((int64_t)E * Cs + kRowWarps - 1) / kRowWarps);
  MOLE_BY_DTYPE(dtype, dispatch_fwd_kernel<T><<<grid, kRowWarps * 32, 0, st>>>(
      static_cast<const T*>(x), counts, offsets, perm, M, E, k, Cs, static_cast<T*>(disp),
      PeerMap{}));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

static int fill_peer_map(PeerMap& pm, void* const* rows, int32_t* const* counts, int n_peers,
                         int rank, int E, const int32_t* all_counts = nullptr) {
  MOLE_REQUIRE(rows != nullptr, "null peer table");
  MOLE_REQUIRE(n_peers >= 2 && n_peers <= kMaxPeers, "peer count %d not in [2, %d]", n_peers, kMaxPeers);
  MOLE_REQUIRE(rank >= 0 && rank < n_peers, "rank %d outside the %d peers", rank, n_peers);
  MOLE_REQUIRE(E % n_peers == 0, "%d experts do not divide over %d ranks", E, n_peers);
  pm = PeerMap{};
  for (int q = 0; q < n_peers; ++q) {
    MOLE_REQUIRE(rows[q] != nullptr, "null buffer for peer %d", q);
    pm.base[q] = rows[q];
    if (counts) {
      MOLE_REQUIRE(counts[q] != nullptr, "null count array for peer %d", q);
      pm.counts[q] = counts[q];
    }
  }
  pm.n = n_peers;
  pm.rank = rank;
  pm.L = E / n_peers;
  pm.all_counts = all_counts;
  pm.E = E;
  return MOLE_OK;
}

// n int32 values of this rank into slot `rank` of every rank's table (peer_tables[q] is rank q's
// [world][n] table mapped into this process): how the ranks tell each other their per-expert row
// counts before a packed dispatch.  One block per destination, plain stores over NVLink.
__global__ void peer_put_kernel(const int32_t* __restrict__ src, int n, const __grid_constant__ PeerMap pm) {
  int32_t* dst = static_cast<int32_t*>(pm.base[blockIdx.x]) + (int64_t)pm.rank * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}

extern "C" int mole_peer_put_i32(const int32_t* src, int32_t n, void* const* peer_tables,
                                 int32_t world, int32_t rank, void* stream) {
  MOLE_REQUIRE(src && peer_tables && n >= 1, "bad argument");
  MOLE_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "rank %d / world %d", rank, world);
  PeerMap pm{};
  for (int q = 0; q < world; ++q) {
    MOLE_REQUIRE(peer_tables[q] != nullptr, "null table of rank %d", q);
    pm.base[q] = peer_tables[q];
  }
  pm.n = world;
  pm.rank = rank;
  peer_put_kernel<<<world, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, n, pm);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_dispatch_fwd_peer(const void* x, const int32_t* counts, const int32_t* offsets,
                                      const int32_t* perm, int64_t T_, int32_t M, int32_t E,
                                      int32_t k, int32_t Cs, int32_t dtype, void* const* peer_rows,
                                      int32_t* const* peer_counts, const int32_t* all_counts,
                                      int32_t n_peers, int32_t rank, void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(x && counts && offsets && perm && (peer_counts || all_counts), "null pointer argument");
  PeerMap pm;
  if (int rc = fill_peer_map(pm, peer_rows, all_counts ? nullptr : peer_counts, n_peers, rank, E, all_counts))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(((int64_t)E * Cs + kRowWarps - 1) / kRowWarps);
  MOLE_BY_DTYPE(dtype, dispatch_fwd_kernel<T><<<grid, kRowWarps * 32, 0, st>>>(
      static_cast<const T*>(x), counts, offsets, perm, M, E, k, Cs, static_cast<T*>(nullptr), pm));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_combine_fwd(const void* rows, const int32_t* idx, const int32_t* slot,
                                const float* gates, int64_t T_, int32_t M, int32_t E, int32_t k,
                                int32_t C, int32_t Cs, int32_t dtype, void* y, void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(rows && idx && slot && gates && y, "null pointer argument");
  MOLE_REQUIRE(C >= 1 && C <= Cs, "capacity %d not in [1, Cs=%d]", C, Cs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((T_ + kRowWarps - 1) / kRowWarps);
  MOLE_BY_DTYPE(dtype, combine_fwd_kernel<T><<<grid, kRowWarps * 32, 0, st>>>(
      static_cast<const T*>(rows), idx, slot, gates, T_, M, k, C, Cs, static_cast<T*>(y)));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_combine_bwd(const void* dy, const void* rows, const float* gates,
                                const int32_t* counts, const int32_t* offsets,
                                const int32_t* perm, int64_t T_, int32_t M, int32_t E, int32_t k,
                                int32_t Cs, int32_t dtype, void* drows, float* dgates,
                                void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(dy && rows && gates && counts && offsets && perm && drows && dgates,
               "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MOLE_CUDA_OK(cudaMemsetAsync(dgates, 0, (size_t)T_ * k * 4, st));
  const unsigned grid = (unsigned)(((int64_t)E * Cs + kRowWarps - 1) / kRowWarps);
  MOLE_BY_DTYPE(dtype, combine_bwd_kernel<T><<<grid, kRowWarps * 32, 0, st>>>(
      static_cast<const T*>(dy), static_cast<const T*>(rows), gates, counts, offsets, perm, M, E,
      k, Cs, static_cast<T*>(drows), dgates, PeerMap{}));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_combine_bwd_peer(const void* dy, const void* rows, const float* gates,
                                     const int32_t* counts, const int32_t* offsets,
                                     const int32_t* perm, int64_t T_, int32_t M, int32_t E,
                                     int32_t k, int32_t Cs, int32_t dtype, void* const* peer_rows,
                                     const int32_t* all_counts, int32_t n_peers, int32_t rank,
                                     float* dgates, void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(dy && rows && gates && counts && offsets && perm && dgates, "null pointer argument");
  PeerMap pm;
  if (int rc = fill_peer_map(pm, peer_rows, nullptr, n_peers, rank, E, all_counts)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MOLE_CUDA_OK(cudaMemsetAsync(dgates, 0, (size_t)T_ * k * 4, st));
  const unsigned grid = (unsigned)(((int64_t)E * Cs + kRowWarps - 1) / kRowWarps);
  MOLE_BY_DTYPE(dtype, combine_bwd_kernel<T><<<grid, kRowWarps * 32, 0, st>>>(
      static_cast<const T*>(dy), static_cast<const T*>(rows), gates, counts, offsets, perm, M, E,
      k, Cs, static_cast<T*>(nullptr), dgates, pm));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

extern "C" int mole_dispatch_bwd(const void* ddisp, const int32_t* idx, const int32_t* slot,
                                 const float* dlogits, const void* wg, int64_t T_, int32_t M,
                                 int32_t E, int32_t k, int32_t C, int32_t Cs, int32_t dtype,
                                 void* dx, void* stream) {
  if (int rc = check_rows(T_, M, E, k, Cs, dtype)) return rc;
  MOLE_REQUIRE(idx && slot && dx, "null pointer argument");
  MOLE_REQUIRE(ddisp || dlogits, "neither ddisp nor dlogits given");
  MOLE_REQUIRE((dlogits == nullptr) == (wg == nullptr), "dlogits and wg must be given together");
  MOLE_REQUIRE(C >= 1 && C <= Cs, "capacity %d not in [1, Cs=%d]", C, Cs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOLE_BF16 && dlogits != nullptr && M % 128 == 0 &&
      ((reinterpret_cast<uintptr_t>(wg) | reinterpret_cast<uintptr_t>(ddisp) |
        reinterpret_cast<uintptr_t>(dx)) & 15) == 0)
    return launch_dispatch_bwd_mma(ddisp, idx, slot, dlogits, wg, T_, M, E, k, C, Cs, dx, st);
  dim3 grid((M + kDbCols - 1) / kDbCols, (unsigned)((T_ + kDbTok - 1) / kDbTok));
  MOLE_BY_DTYPE(dtype, dispatch_bwd_kernel<T><<<grid, 256, 0, st>>>(
      static_cast<const T*>(ddisp), idx, slot, dlogits, static_cast<const T*>(wg), T_, M, E, k, C,
      Cs, static_cast<T*>(dx)));
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}
