// Adam step for offloaded experts on the GPU ("instant Adam": MOLE/cpp/core.cpp:848-943, called
// right after an offloaded expert batch's backward, core.cpp:1216-1227) and the greedy
// assignment of spare pool slots to prefetches across layers (MOLE/cpp/core.cpp:1302-1345).
//
// The reference runs the update as about ten ATen elementwise kernels per tensor
// (MOLE/cpp/define.hpp:543-579), each a full pass over p, m, v or g.  Here it is one pass: p, m,
// v and g are read once, p, m and v written once (HBM-bound, 7 accesses of n elements).
#include <cmath>

#include "common.cuh"

namespace mole {

struct AdamScalars {
  float beta1, beta2, lr, lam, eps;
  float inv_bias1, inv_bias2;      // 1 / (1 - beta^t) with t already advanced
  int adamw;
};

// Arithmetic of MOLE/cpp/define.hpp:552-566, in fp32 whatever the storage type:
//   adamW: p *= 1 - lam lr;   else: g += lam p
//   m = b1 m + (1 - b1) g;  v = b2 v + (1 - b2) g g
//   p -= lr (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)
__device__ __forceinline__ void adam_one(float& p, float& m, float& v, float g, const AdamScalars& a) {
  if (a.adamw) p = p * (1.0f - a.lam * a.lr);
  else g = g + a.lam * p;
  m = a.beta1 * m + (1.0f - a.beta1) * g;
  v = a.beta2 * v + (1.0f - a.beta2) * g * g;
  const float mt = m * a.inv_bias1;
  const float vt = v * a.inv_bias2;
  p = p - a.lr * mt / (sqrtf(vt) + a.eps);
}

template <typename T>
__global__ void __launch_bounds__(256)
adam_kernel(T* __restrict__ p, T* __restrict__ m, T* __restrict__ v, const T* __restrict__ g,
            const T* __restrict__ g2, int64_t n, AdamScalars a) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float pv[V], mv[V], vv[V], gv[V];
    Vec16<T>::load(p + i * V, pv);
    Vec16<T>::load(m + i * V, mv);
    Vec16<T>::load(v + i * V, vv);
    Vec16<T>::load(g + i * V, gv);
    if (g2 != nullptr) {             // gradient accumulated over earlier micro-steps (core.cpp:906-918)
      float hv[V];
      Vec16<T>::load(g2 + i * V, hv);
#pragma unroll
      for (int j = 0; j < V; ++j) gv[j] += hv[j];
    }
#pragma unroll
    for (int j = 0; j < V; ++j) adam_one(pv[j], mv[j], vv[j], gv[j], a);
    Vec16<T>::store(p + i * V, pv);
    Vec16<T>::store(m + i * V, mv);
    Vec16<T>::store(v + i * V, vv);
  }
  // tail (n not a multiple of the vector width)
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float pp = Elem<T>::to_f(p[i]), mm = Elem<T>::to_f(m[i]), vv = Elem<T>::to_f(v[i]);
    float gg = Elem<T>::to_f(g[i]);
    if (g2 != nullptr) gg += Elem<T>::to_f(g2[i]);
    adam_one(pp, mm, vv, gg, a);
    p[i] = Elem<T>::from_f(pp);
    m[i] = Elem<T>::from_f(mm);
    v[i] = Elem<T>::from_f(vv);
  }
}

}  // namespace mole

using namespace mole;

extern "C" int mole_adam_update(void* p, void* m, void* v, const void* g, const void* g_extra,
                                int64_t n, int32_t dtype, float beta1, float beta2, int32_t t,
                                float lr, float lam, float eps, int32_t adamw, void* stream) {
  MOLE_REQUIRE(p && m && v && g, "null pointer argument");
  MOLE_REQUIRE(n >= 0, "n=%lld", (long long)n);
  MOLE_REQUIRE(t >= 1, "step count t=%d must be at least 1 (the count after this step)", t);
  MOLE_REQUIRE(dtype == MOLE_F32 || dtype == MOLE_BF16, "dtype %d", dtype);
  for (const void* q : {(const void*)p, (const void*)m, (const void*)v, g, g_extra})
    MOLE_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0, "pointer %p not 16-byte aligned", q);
  if (n == 0) return MOLE_OK;
  AdamScalars a;
  a.beta1 = beta1; a.beta2 = beta2; a.lr = lr; a.lam = lam; a.eps = eps; a.adamw = adamw;
  a.inv_bias1 = (float)(1.0 / (1.0 - std::pow((double)beta1, (double)t)));
  a.inv_bias2 = (float)(1.0 / (1.0 - std::pow((double)beta2, (double)t)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vec = dtype == MOLE_F32 ? 4 : 8;
  int64_t blocks = (n / vec + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (dtype == MOLE_F32)
    adam_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<float*>(p), static_cast<float*>(m), static_cast<float*>(v),
        static_cast<const float*>(g), static_cast<const float*>(g_extra), n, a);
  else
    adam_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<__nv_bfloat16*>(p), static_cast<__nv_bfloat16*>(m),
        static_cast<__nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(g),
        static_cast<const __nv_bfloat16*>(g_extra), n, a);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// Greedy assignment of prefetches to pool slots across layers.  Layer i can overlap F[i]
// expert fetches with the time before it runs and owns E[i] offloaded experts; P slots are
// free.  A layer that could fetch more than it owns lends the surplus ("global prefetch": it
// fetches for later layers while it runs); later layers that cannot cover their own experts
// take from the most recent lender first (a stack).  Outputs: local[i] = experts layer i
// prefetches for itself; triples (lender, borrower, count).
extern "C" int mole_fast_assign_prefetch(int32_t P, const int32_t* F, const int32_t* E, int32_t n,
                                         int32_t* local, int32_t* triples, int32_t capacity,
                                         int32_t* n_triples) {
  MOLE_REQUIRE(F && E && local && n_triples && n >= 0 && P >= 0, "bad argument");
  struct Lend { int layer, left; };
  Lend stack[1024];
  int depth = 0, nt = 0, p_cur = P;
  MOLE_REQUIRE(n <= 1024, "at most 1024 layers");
  for (int i = 0; i < n; ++i) {
    const int fetchable = p_cur < F[i] ? p_cur : F[i];
    if (fetchable <= E[i]) {
      int need = E[i] - fetchable;
      local[i] = fetchable;
      while (depth > 0 && need > 0) {
        Lend& top = stack[depth - 1];
        const int take = top.left > need ? need : top.left;
        if (triples && nt < capacity) {
          triples[3 * nt] = top.layer; triples[3 * nt + 1] = i; triples[3 * nt + 2] = take;
        }
        ++nt;
        p_cur += take;
        need -= take;
        top.left -= take;
        if (top.left == 0) --depth;
      }
    } else {
      const int lend = fetchable - E[i];
      p_cur -= lend;
      stack[depth].layer = i; stack[depth].left = lend;
      ++depth;
      local[i] = E[i];
    }
  }
  *n_triples = nt;
  return MOLE_OK;
}
