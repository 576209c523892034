// Tile schedule, CUDA-core grouped GEMM (exact fp32 accumulation) and per-expert column sums.
//
// The CUDA-core GEMM is what the fp32 layer runs on: tcgen05 has no fp32-precision input type
// (kind::tf32 keeps 10 mantissa bits), and the reference computes the FFN in fp32
// (MOLE/cpp/core.cpp:350-353 on float tensors).  It follows the same schedule and epilogues
// as the tensor-core back end.
#include "gemm.cuh"

namespace mole {

// ---- schedule -----------------------------------------------------------------------
int64_t schedule_bytes(int L, int n_src, int Cs) {
  const int64_t max_tiles = (int64_t)L * n_src * (Cs / kTileRows);
  return (1 + 2 * (L + 1) + 3 * max_tiles + 16) * 4;
}
Schedule carve_schedule(void* ws, int L, int n_src, int Cs) {
  Schedule s;
  int32_t* p = static_cast<int32_t*>(ws);
  s.max_tiles = L * n_src * (Cs / kTileRows);
  s.n_tiles = p;
  s.expert_tile_start = p + 4;
  s.expert_pair_start = s.expert_tile_start + (L + 1);
  s.tile_row0 = s.expert_pair_start + (L + 1) + 3;
  s.tile_expert = s.tile_row0 + s.max_tiles;
  s.tile_rows = s.tile_expert + s.max_tiles;
  return s;
}

// One block.  Pairs (l, w) in expert-major order; pair p contributes ceil(count/128) tiles.
__global__ void __launch_bounds__(256)
schedule_kernel(const int32_t* __restrict__ counts, int L, int n_src, int Cs, int e_begin,
                int e_end, Schedule s) {
  __shared__ int part[256];
  __shared__ int est[kMaxLocalExperts + 1];      // expert_tile_start, for the pair prefix below
  const int tid = threadIdx.x;
  const int npairs = (e_end - e_begin) * n_src;
  const int per = (npairs + 255) / 256;
  const int p0 = tid * per, p1 = min(npairs, p0 + per);
  int sum = 0;
  for (int p = p0; p < p1; ++p) {
    const int l = e_begin + p / n_src, w = p % n_src;
    sum += (min(counts[w * L + l], Cs) + kTileRows - 1) / kTileRows;
  }
  part[tid] = sum;
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int i = 0; i < 256; ++i) { const int v = part[i]; part[i] = run; run += v; }
    *s.n_tiles = run;
    s.expert_tile_start[e_end - e_begin] = run;
    est[e_end - e_begin] = run;
  }
  __syncthreads();
  int t = part[tid];
  for (int p = p0; p < p1; ++p) {
    const int l = e_begin + p / n_src, w = p % n_src;
    if (w == 0) { s.expert_tile_start[l - e_begin] = t; est[l - e_begin] = t; }
    const int cnt = min(counts[w * L + l], Cs);
    const int nt = (cnt + kTileRows - 1) / kTileRows;
    const int row0 = (w * L + l) * Cs;
    for (int i = 0; i < nt; ++i) {
      s.tile_row0[t + i] = row0 + i * kTileRows;
      s.tile_expert[t + i] = l;
      s.tile_rows[t + i] = min(kTileRows, cnt - i * kTileRows);
    }
    t += nt;
  }
  __syncthreads();
  if (tid == 0) {
    const int ne = e_end - e_begin;
    int run = 0;
    for (int i = 0; i < ne; ++i) {
      s.expert_pair_start[i] = run;
      run += (est[i + 1] - est[i] + 1) / 2;
    }
    s.expert_pair_start[ne] = run;
  }
}

int build_schedule(const int32_t* counts, int L, int n_src, int Cs, int e_begin, int e_end,
                   Schedule s, cudaStream_t st) {
  schedule_kernel<<<1, 256, 0, st>>>(counts, L, n_src, Cs, e_begin, e_end, s);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// ---- per-expert compaction (several source ranks per expert) -------------------------------
// The exchange leaves expert l's rows in n_src chunks [w][l][Cs], each with its own ragged last
// tile.  The compacted layout is [l][n_src * Cs]: the expert's valid rows of all sources packed at
// the front of its region (source order), zero rows up to the next multiple of 128.  One ragged
// tile per expert instead of one per (source, expert): at 8 source ranks x ~256 rows that is 17
// tiles instead of 20-24.  The region of an expert does not depend on which experts a call covers.
__global__ void __launch_bounds__(256)
schedule_compact_kernel(const int32_t* __restrict__ counts, int L, int n_src, int Cs, int e_begin,
                        int e_end, Schedule s) {
  __shared__ int tiles[256];
  const int tid = threadIdx.x;
  const int ne = e_end - e_begin;
  int nt = 0, rows = 0;
  if (tid < ne) {
    for (int w = 0; w < n_src; ++w) rows += min(counts[w * L + e_begin + tid], Cs);
    nt = (rows + kTileRows - 1) / kTileRows;
  }
  tiles[tid] = nt;
  __syncthreads();
  if (tid == 0) {
    int run = 0, pairs = 0;
    for (int i = 0; i < ne; ++i) {
      s.expert_tile_start[i] = run;
      s.expert_pair_start[i] = pairs;
      run += tiles[i];
      pairs += (tiles[i] + 1) / 2;
    }
    s.expert_tile_start[ne] = run;
    s.expert_pair_start[ne] = pairs;
    *s.n_tiles = run;
  }
  __syncthreads();
  if (tid < ne) {
    const int t0 = s.expert_tile_start[tid];
    const int row0 = (e_begin + tid) * n_src * Cs;
    for (int i = 0; i < nt; ++i) {
      s.tile_row0[t0 + i] = row0 + i * kTileRows;
      s.tile_expert[t0 + i] = e_begin + tid;
      s.tile_rows[t0 + i] = min(kTileRows, rows - i * kTileRows);
    }
  }
}

// One warp per row of the compacted layout: finds the (source, slot) the row comes from, records
// it in rowmap (when given) and copies the row; pad rows are zeroed and mapped to -1.  With
// src == nullptr the rows are already where they belong (the senders packed them): only the row
// map is written and the pad rows are zeroed.
template <typename T>
__global__ void __launch_bounds__(256)
compact_gather_kernel(const T* __restrict__ src, const int32_t* __restrict__ counts, int L,
                      int n_src, int Cs, int e_begin, int e_end, int width,
                      T* __restrict__ dst, int32_t* __restrict__ rowmap) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);      // row inside the range
  const int region = n_src * Cs;
  if (r >= (int64_t)(e_end - e_begin) * region) return;
  const int l = e_begin + (int)(r / region);
  int j = (int)(r % region);
  int total = 0;
  for (int w = 0; w < n_src; ++w) total += min(counts[w * L + l], Cs);
  const int padded = (total + kTileRows - 1) / kTileRows * kTileRows;
  if (j >= padded) return;
  const int64_t drow = (int64_t)l * region + j;
  int64_t srow = -1;
  if (j < total) {
    for (int w = 0; w < n_src; ++w) {
      const int c = min(counts[w * L + l], Cs);
      if (j < c) { srow = ((int64_t)w * L + l) * Cs + j; break; }
      j -= c;
    }
  }
  if (rowmap != nullptr && lane == 0) rowmap[drow] = (int32_t)srow;
  uint4* d4 = reinterpret_cast<uint4*>(dst + drow * width);
  const int nvec = width / Vec16<T>::N;
  if (srow < 0) {
    for (int i = lane; i < nvec; i += 32) d4[i] = make_uint4(0, 0, 0, 0);
  } else if (src != nullptr) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src + srow * width);
    for (int i = lane; i < nvec; i += 32) d4[i] = __ldg(s4 + i);
  }
}

int build_schedule_compact(const int32_t* counts, int L, int n_src, int Cs, int e_begin, int e_end,
                           Schedule s, cudaStream_t st) {
  schedule_compact_kernel<<<1, 256, 0, st>>>(counts, L, n_src, Cs, e_begin, e_end, s);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

int compact_gather(int dtype, const void* src, const int32_t* counts, int L, int n_src, int Cs,
                   int e_begin, int e_end, int width, void* dst, int32_t* rowmap, cudaStream_t st) {
  const int64_t rows = (int64_t)(e_end - e_begin) * n_src * Cs;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == MOLE_F32)
    compact_gather_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), counts, L, n_src,
                                                       Cs, e_begin, e_end, width,
                                                       static_cast<float*>(dst), rowmap);
  else
    compact_gather_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(src), counts, L, n_src, Cs, e_begin, e_end, width,
        static_cast<__nv_bfloat16*>(dst), rowmap);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// ---- CUDA-core row-grouped GEMM -------------------------------------------------------
constexpr int kSB = 64;    // block tile 64 x 64
constexpr int kSK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
simt_row_gemm_kernel(const __grid_constant__ RowGemmArgs a) {
  __shared__ float As[kSK][kSB + 4];
  __shared__ float Bs[kSK][kSB + 4];
  const int tile = blockIdx.y >> 1, half = blockIdx.y & 1;
  if (tile >= *a.sched.n_tiles) return;
  const int row0 = a.sched.tile_row0[tile] + half * kSB;
  const int e = a.sched.tile_expert[tile];
  const int slot = a.wslot.s[e];
  const int n0 = blockIdx.x * kSB;
  const T* A = static_cast<const T*>(a.A);
  const T* W = static_cast<const T*>(a.W) + (int64_t)slot * a.w_expert_stride;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int K = a.K, N = a.N;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kSK) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = tid + 256 * r;             // 1024 elements of each tile
      {                                        // A tile: 64 rows x 16 k, k fastest
        const int rr = i >> 4, kk = i & 15;
        As[kk][rr] = Elem<T>::to_f(A[(int64_t)(row0 + rr) * K + k0 + kk]);
      }
      if (a.w_nk) {                            // W_e[n][k], k fastest
        const int nn = i >> 4, kk = i & 15;
        Bs[kk][nn] = Elem<T>::to_f(W[(int64_t)(n0 + nn) * K + k0 + kk]);
      } else {                                 // W_e[k][n], n fastest
        const int kk = i >> 6, nn = i & 63;
        Bs[kk][nn] = Elem<T>::to_f(W[(int64_t)(k0 + kk) * N + n0 + nn]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }
  const T* bias = a.bias ? static_cast<const T*>(a.bias) + (int64_t)slot * N : nullptr;
  const T* aux = static_cast<const T*>(a.aux);
  T* out0 = static_cast<T*>(a.out0);
  T* out1 = static_cast<T*>(a.out1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      const float bv = bias ? Elem<T>::to_f(bias[n]) : 0.f;
      const float xv = a.epi == EPI_DACT ? Elem<T>::to_f(aux[r * N + n]) : 0.f;
      const EpiOut o = epilogue_apply(a.epi, acc[i][j], bv, xv, a.act, a.gelu_bwd);
      const T stored = Elem<T>::from_f(o.v0);
      out0[r * N + n] = stored;
      // the activation is taken of the stored (rounded) pre-activation, the value backward sees
      if (a.epi == EPI_FC1) out1[r * N + n] = Elem<T>::from_f(act_fwd(Elem<T>::to_f(stored), a.act));
    }
  }
}

// out_e[p, q] (+)= sum_r A[r, p] * B[r, q] over the expert's tiles.
template <typename T>
__global__ void __launch_bounds__(256)
simt_wgrad_kernel(const __grid_constant__ WgradArgs a) {
  __shared__ float As[kSK][kSB + 4];
  __shared__ float Bs[kSK][kSB + 4];
  const int el = blockIdx.z;
  const int t0 = a.sched.expert_tile_start[el], t1 = a.sched.expert_tile_start[el + 1];
  const int e = a.e_begin + el;
  const int slot = a.gslot.s[e];
  const int q0 = blockIdx.x * kSB, p0 = blockIdx.y * kSB;
  const T* A = static_cast<const T*>(a.A);
  const T* B = static_cast<const T*>(a.B);
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int P = a.P, Q = a.Q;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int t = t0; t < t1; ++t) {
    const int64_t row0 = a.sched.tile_row0[t];
    for (int r0 = 0; r0 < kTileRows; r0 += kSK) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = tid + 256 * r;
        const int kk = i >> 6, cc = i & 63;
        As[kk][cc] = Elem<T>::to_f(A[(row0 + r0 + kk) * P + p0 + cc]);
        Bs[kk][cc] = Elem<T>::to_f(B[(row0 + r0 + kk) * Q + q0 + cc]);
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kSK; ++kk) {
        const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
        const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
  T* out = static_cast<T*>(a.out) + (int64_t)slot * P * Q;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t o = (int64_t)(p0 + ty * 4 + i) * Q + q0 + tx * 4 + j;
      float v = acc[i][j];
      if (a.accumulate) v += Elem<T>::to_f(out[o]);
      out[o] = Elem<T>::from_f(v);
    }
}

// Block: 8 column groups of one 16-byte vector (a row segment of 128 bytes) x 32 row lanes; one
// expert.  Every thread keeps four 16-byte loads in flight.  Narrow column blocks keep the grid
// large when a rank owns few experts with many rows each (8 experts x 2048 rows on eight GPUs: a
// 256-column block per expert left 64 blocks for 148 SMs, each walking 2048 rows).
constexpr int kCsCG = 8, kCsRL = 32;
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const __grid_constant__ ColsumArgs a) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[kCsRL][kCsCG * V + 1];
  const int el = blockIdx.y;
  const int t0 = a.sched.expert_tile_start[el], t1 = a.sched.expert_tile_start[el + 1];
  const int slot = a.gslot.s[a.e_begin + el];
  const int cg = threadIdx.x % kCsCG, rl = threadIdx.x / kCsCG;
  const int col = (blockIdx.x * kCsCG + cg) * V;
  const T* A = static_cast<const T*>(a.A);
  float s[V];
#pragma unroll
  for (int c = 0; c < V; ++c) s[c] = 0.f;
  if (col < a.N) {
    for (int t = t0; t < t1; ++t) {
      const T* base = A + ((int64_t)a.sched.tile_row0[t] + rl) * a.N + col;
      const int valid = a.sched.tile_rows[t];               // rows beyond it may never have been written
      // rows rl + {0, 32, 64, 96} of the tile (kTileRows = 4 * kCsRL)
      float v[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (kCsRL * u + rl < valid) {
          Vec16<T>::load(base + (int64_t)(kCsRL * u) * a.N, v[u]);
        } else {
#pragma unroll
          for (int c = 0; c < V; ++c) v[u][c] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int c = 0; c < V; ++c) s[c] += v[u][c];
    }
  }
#pragma unroll
  for (int c = 0; c < V; ++c) red[rl][cg * V + c] = s[c];
  __syncthreads();
  for (int i = threadIdx.x; i < kCsCG * V; i += 256) {
    const int n = blockIdx.x * kCsCG * V + i;
    if (n < a.N) {
      float v = 0.f;
#pragma unroll
      for (int r = 0; r < kCsRL; ++r) v += red[r][i];
      T* out = static_cast<T*>(a.out) + (int64_t)slot * a.N + n;
      if (a.accumulate) v += Elem<T>::to_f(*out);
      *out = Elem<T>::from_f(v);
    }
  }
}

int simt_row_gemm(int dtype, const RowGemmArgs& a, cudaStream_t st) {
  MOLE_REQUIRE(a.N % kSB == 0 && a.K % kSK == 0, "CUDA-core GEMM needs N %% 64 == 0, K %% 16 == 0");
  MOLE_REQUIRE(a.sched.max_tiles * 2 <= 65535, "too many row tiles for the CUDA-core GEMM grid");
  MOLE_REQUIRE(a.rowmap == nullptr, "the CUDA-core GEMM does not scatter its output rows");
  dim3 grid(a.N / kSB, a.sched.max_tiles * 2);
  if (dtype == MOLE_F32) simt_row_gemm_kernel<float><<<grid, 256, 0, st>>>(a);
  else simt_row_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

int simt_wgrad(int dtype, const WgradArgs& a, cudaStream_t st) {
  MOLE_REQUIRE(a.P % kSB == 0 && a.Q % kSB == 0, "CUDA-core wgrad needs F, M %% 64 == 0");
  if (a.n_experts <= 0) return MOLE_OK;
  dim3 grid(a.Q / kSB, a.P / kSB, a.n_experts);
  if (dtype == MOLE_F32) simt_wgrad_kernel<float><<<grid, 256, 0, st>>>(a);
  else simt_wgrad_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

int colsum(int dtype, const ColsumArgs& a, cudaStream_t st) {
  const int vec = dtype == MOLE_F32 ? 4 : 8;
  MOLE_REQUIRE(a.N % vec == 0, "column sums need 16-byte rows");
  if (a.n_experts <= 0) return MOLE_OK;
  static_assert(kTileRows == 4 * kCsRL, "a thread takes four rows of a tile");
  dim3 grid((a.N + kCsCG * vec - 1) / (kCsCG * vec), a.n_experts);
  if (dtype == MOLE_F32) colsum_kernel<float><<<grid, 256, 0, st>>>(a);
  else colsum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

}  // namespace mole
