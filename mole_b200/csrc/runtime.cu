// Runtime services behind the C ABI: error strings, the device fault word, the stream set,
// the NCCL all-to-all and the offloaded-expert slot pool.
//
//   streams  <- MOLE/cpp/stream.cpp:38-144, 156-205   (16 streams, roles 1..4, wait helpers)
//   comm     <- MOLE/cpp/communication.cpp:49-100     (own communicator, grouped send/recv)
//   pool     <- MOLE/cpp/umemory.cpp:92-205, MOLE/cpp/define.hpp:143-193 (slots, prefetch stack,
//               slot -> last-user ordering), MOLE/cpp/uparameter.cpp:58-71, MOLE/cpp/transfer.cu
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace mole {

char* last_error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

// One fault word per device (256 bytes of device memory, allocated at the device's first use).
struct FaultSlot {
  int32_t* word = nullptr;        // device
  int32_t* host = nullptr;        // pinned: where mole_device_fault_poll copies the word
  cudaEvent_t polled = nullptr;   // recorded behind the last poll's copy
  bool poll_pending = false;
};
static FaultSlot g_fault[kMaxDevices];
static std::mutex g_fault_mu;
static FaultSlot* fault_slot() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_fault_mu);
  FaultSlot& f = g_fault[dev];
  if (!f.word) {
    if (cudaMalloc(&f.word, 256) != cudaSuccess) { f.word = nullptr; return nullptr; }
    cudaMemset(f.word, 0, 256);
    if (cudaMallocHost(&f.host, 64) != cudaSuccess) f.host = nullptr;
    else *f.host = 0;
    if (cudaEventCreateWithFlags(&f.polled, cudaEventDisableTiming) != cudaSuccess) f.polled = nullptr;
  }
  return &f;
}
int32_t* device_fault_word() {
  FaultSlot* f = fault_slot();
  return f ? f->word : nullptr;
}

int sm_count() {
  static PerDeviceInt n;
  const int dev = current_device();
  int64_t v = n.get(dev);
  if (v == 0) {
    int a = 0;
    cudaDeviceGetAttribute(&a, cudaDevAttrMultiProcessorCount, dev);
    v = a > 0 ? a : 148;
    n.set(dev, v);
  }
  return (int)v;
}

static std::atomic<int64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct ProfileEntry { cudaEvent_t a, b; int kind; };
static bool g_profile = false;
static std::vector<ProfileEntry> g_entries;
bool profile_enabled() { return g_profile; }
void profile_begin(cudaStream_t st, int kind) {
  ProfileEntry e;
  e.kind = kind;
  if (cudaEventCreate(&e.a) != cudaSuccess || cudaEventCreate(&e.b) != cudaSuccess) return;
  cudaEventRecord(e.a, st);
  g_entries.push_back(e);
}
void profile_end(cudaStream_t st) {
  if (!g_entries.empty()) cudaEventRecord(g_entries.back().b, st);
}

}  // namespace mole

using namespace mole;

extern "C" int mole_launch_count(int64_t* n) {
  MOLE_REQUIRE(n != nullptr, "n is null");
  *n = g_launches.load();
  return MOLE_OK;
}
extern "C" int mole_profile_gemm(int32_t enable) {
  g_profile = enable != 0;
  return MOLE_OK;
}
extern "C" int mole_profile_read(float* ms, int32_t* kind, int32_t capacity, int32_t* n) {
  MOLE_REQUIRE(n != nullptr, "n is null");
  *n = (int)g_entries.size();
  for (size_t i = 0; i < g_entries.size(); ++i) {
    ProfileEntry& e = g_entries[i];
    float t = 0.f;
    MOLE_CUDA_OK(cudaEventSynchronize(e.b));
    MOLE_CUDA_OK(cudaEventElapsedTime(&t, e.a, e.b));
    if (ms && kind && (int)i < capacity) { ms[i] = t; kind[i] = e.kind; }
    cudaEventDestroy(e.a);
    cudaEventDestroy(e.b);
  }
  g_entries.clear();
  return MOLE_OK;
}

extern "C" int mole_version(void) { return 100; }
extern "C" const char* mole_last_error_string(void) { return last_error_buffer(); }
extern "C" int64_t mole_capacity_stride(int64_t capacity) {
  return (capacity + kTileRows - 1) / kTileRows * kTileRows;
}
extern "C" int mole_device_fault(void* stream, int32_t* fault) {
  MOLE_REQUIRE(fault != nullptr, "fault is null");
  int32_t* w = device_fault_word();
  if (!w) return fail(MOLE_ERR_CUDA, "fault word not allocated");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MOLE_CUDA_OK(cudaMemcpyAsync(fault, w, 4, cudaMemcpyDeviceToHost, st));
  MOLE_CUDA_OK(cudaStreamSynchronize(st));
  if (*fault != 0) MOLE_CUDA_OK(cudaMemsetAsync(w, 0, 4, st));
  return MOLE_OK;
}
// The same check without a host wait: poll enqueues a copy of the word into pinned host memory
// behind the work already on `stream`; peek returns the last copy that has landed.
// The word travels by a one-thread kernel that stores it into the pinned (device-visible) host
// word: a 4-byte copy by the DMA engine in the middle of the compute stream cost ~20 us of
// stream time (the copy and the engine switch around it), this is an ordinary tiny launch.
__global__ void fault_word_to_host_kernel(const int32_t* __restrict__ word, volatile int32_t* host) {
  *host = *word;
}

extern "C" int mole_device_fault_poll(void* stream) {
  FaultSlot* f = fault_slot();
  if (!f || !f->host || !f->polled) return fail(MOLE_ERR_CUDA, "fault word not allocated");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // A stream that is being captured into a CUDA graph takes no poll: the event of the copy would
  // become part of the graph and could no longer be queried.  Whoever replays the graph polls
  // behind a replay instead.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return MOLE_OK;
  if (f->poll_pending && cudaEventQuery(f->polled) != cudaSuccess) {
    cudaGetLastError();           // the previous poll's copy is still in flight: keep that one
    return MOLE_OK;
  }
  fault_word_to_host_kernel<<<1, 1, 0, st>>>(f->word, f->host + 1);
  MOLE_LAUNCH_OK();
  MOLE_CUDA_OK(cudaEventRecord(f->polled, st));
  f->poll_pending = true;
  return MOLE_OK;
}
extern "C" int mole_device_fault_peek(int32_t* fault) {
  MOLE_REQUIRE(fault != nullptr, "fault is null");
  FaultSlot* f = fault_slot();
  if (!f || !f->host || !f->polled) return fail(MOLE_ERR_CUDA, "fault word not allocated");
  if (f->poll_pending && cudaEventQuery(f->polled) == cudaSuccess) {
    f->host[0] = f->host[1];
    f->poll_pending = false;
  } else {
    cudaGetLastError();
  }
  *fault = f->host[0];
  return MOLE_OK;
}

// ---- streams --------------------------------------------------------------------------
constexpr int kStreams = 16;
constexpr int kEventRing = 64;
constexpr int kTicketRing = 1024;
struct mole_ctx {
  int device;
  int single;
  cudaStream_t streams[kStreams];
  cudaEvent_t ring[kEventRing];
  int ring_pos;
  cudaEvent_t tickets[kTicketRing];     // per-record edges (mole_ctx_event_record / _wait)
  int64_t ticket_serial[kTicketRing];   // which record call last used the slot
  int64_t next_ticket;
};

static cudaEvent_t next_event(mole_ctx* c) {
  cudaEvent_t e = c->ring[c->ring_pos];
  c->ring_pos = (c->ring_pos + 1) % kEventRing;
  return e;
}

extern "C" int mole_ctx_create(int32_t device, int32_t single_stream, mole_ctx** out) {
  MOLE_REQUIRE(out != nullptr, "ctx out-pointer is null");
  MOLE_CUDA_OK(cudaSetDevice(device));
  mole_ctx* c = new mole_ctx();
  c->device = device;
  c->single = single_stream;
  c->ring_pos = 0;
  for (int i = 0; i < kStreams; ++i) {
    c->streams[i] = nullptr;            // single-stream mode: every role is the default stream
    if (!single_stream) MOLE_CUDA_OK(cudaStreamCreateWithFlags(&c->streams[i], cudaStreamNonBlocking));
  }
  for (int i = 0; i < kEventRing; ++i)
    MOLE_CUDA_OK(cudaEventCreateWithFlags(&c->ring[i], cudaEventDisableTiming));
  for (int i = 0; i < kTicketRing; ++i) {
    MOLE_CUDA_OK(cudaEventCreateWithFlags(&c->tickets[i], cudaEventDisableTiming));
    c->ticket_serial[i] = -1;
  }
  c->next_ticket = 0;
  *out = c;
  return MOLE_OK;
}
extern "C" int mole_ctx_destroy(mole_ctx* c) {
  if (!c) return MOLE_OK;
  for (int i = 0; i < kStreams; ++i)
    if (c->streams[i]) cudaStreamDestroy(c->streams[i]);
  for (int i = 0; i < kEventRing; ++i) cudaEventDestroy(c->ring[i]);
  for (int i = 0; i < kTicketRing; ++i) cudaEventDestroy(c->tickets[i]);
  delete c;
  return MOLE_OK;
}
extern "C" int mole_ctx_stream(mole_ctx* c, int32_t idx, void** stream) {
  MOLE_REQUIRE(c && stream, "null argument");
  MOLE_REQUIRE(idx >= 0 && idx < kStreams, "stream index %d outside [0,%d)", idx, kStreams);
  *stream = c->streams[idx];
  return MOLE_OK;
}
extern "C" int mole_ctx_wait(mole_ctx* c, void* waiter, void* waited) {
  MOLE_REQUIRE(c != nullptr, "ctx is null");
  if (waiter == waited) return MOLE_OK;
  cudaEvent_t e = next_event(c);
  MOLE_CUDA_OK(cudaEventRecord(e, static_cast<cudaStream_t>(waited)));
  MOLE_CUDA_OK(cudaStreamWaitEvent(static_cast<cudaStream_t>(waiter), e, 0));
  return MOLE_OK;
}
// Per-record edges: what the reference keeps as comp_event / comm_event / para_event in every
// _BatchRecord (MOLE/cpp/define.hpp:634-636, recorded at MOLE/cpp/core.cpp:177).  A ticket names
// the work enqueued on `stream` up to the record call; a later wait orders another stream behind
// exactly that work, not behind everything the first stream has been given since.
extern "C" int mole_ctx_event_record(mole_ctx* c, void* stream, int64_t* ticket) {
  MOLE_REQUIRE(c && ticket, "null argument");
  const int64_t t = c->next_ticket++;
  const int slot = (int)(t % kTicketRing);
  MOLE_CUDA_OK(cudaEventRecord(c->tickets[slot], static_cast<cudaStream_t>(stream)));
  c->ticket_serial[slot] = t;
  *ticket = t;
  return MOLE_OK;
}
extern "C" int mole_ctx_event_wait(mole_ctx* c, int64_t ticket, void* stream) {
  MOLE_REQUIRE(c != nullptr, "ctx is null");
  MOLE_REQUIRE(ticket >= 0 && ticket < c->next_ticket, "ticket %lld was never issued", (long long)ticket);
  const int slot = (int)(ticket % kTicketRing);
  if (c->ticket_serial[slot] != ticket)
    return fail(MOLE_ERR_STATE, "ticket %lld is older than the last %d records and has been reused",
                (long long)ticket, kTicketRing);
  MOLE_CUDA_OK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), c->tickets[slot], 0));
  return MOLE_OK;
}
extern "C" int mole_ctx_synchronize(mole_ctx* c, int32_t idx) {
  MOLE_REQUIRE(c != nullptr, "ctx is null");
  MOLE_REQUIRE(idx >= 0 && idx < kStreams, "stream index %d outside [0,%d)", idx, kStreams);
  MOLE_CUDA_OK(cudaStreamSynchronize(c->streams[idx]));
  return MOLE_OK;
}
extern "C" int mole_store_to_host(mole_ctx* c, void* host_dst, const void* dev_src, int64_t bytes,
                                  void* after_stream) {
  MOLE_REQUIRE(c && host_dst && dev_src && bytes >= 0, "bad argument");
  cudaStream_t back = c->streams[4];
  if (int rc = mole_ctx_wait(c, back, after_stream)) return rc;
  MOLE_CUDA_OK(cudaMemcpyAsync(host_dst, dev_src, (size_t)bytes, cudaMemcpyDeviceToHost, back));
  return MOLE_OK;
}

// ---- NCCL, bound at first use from the libnccl the process already has -------------------
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  const char* (*GetErrorString)(ncclResult_t);
  bool ok;
};
static NcclApi* nccl_api() {
  static NcclApi api{};
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
#define MOLE_BIND(name) \
  api.name = reinterpret_cast<decltype(api.name)>(dlsym(h, "nccl" #name)); \
  if (!api.name) return;
    MOLE_BIND(GetUniqueId) MOLE_BIND(CommInitRank) MOLE_BIND(CommDestroy) MOLE_BIND(GroupStart)
    MOLE_BIND(GroupEnd) MOLE_BIND(Send) MOLE_BIND(Recv) MOLE_BIND(GetErrorString)
#undef MOLE_BIND
    api.ok = true;
  });
  return api.ok ? &api : nullptr;
}
#define MOLE_NCCL_OK(api, expr)                                                        \
  do {                                                                                 \
    ncclResult_t _r = (expr);                                                          \
    if (_r != ncclSuccess)                                                             \
      return fail(MOLE_ERR_NCCL, "%s -> %s", #expr, (api)->GetErrorString(_r));        \
  } while (0)

struct mole_comm {
  ncclComm_t comm;
  int world, rank, device;
};

extern "C" int mole_comm_unique_id(uint8_t* id128) {
  MOLE_REQUIRE(id128 != nullptr, "id buffer is null");
  NcclApi* n = nccl_api();
  if (!n) return fail(MOLE_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
  static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
  ncclUniqueId id;
  MOLE_NCCL_OK(n, n->GetUniqueId(&id));
  memcpy(id128, &id, 128);
  return MOLE_OK;
}
extern "C" int mole_comm_create(const uint8_t* id128, int32_t world_size, int32_t rank,
                                int32_t device, mole_comm** out) {
  MOLE_REQUIRE(id128 && out, "null argument");
  MOLE_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size, "rank %d / world %d", rank, world_size);
  NcclApi* n = nccl_api();
  if (!n) return fail(MOLE_ERR_NCCL, "libnccl.so.2 could not be loaded");
  MOLE_CUDA_OK(cudaSetDevice(device));
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  mole_comm* c = new mole_comm();
  c->world = world_size; c->rank = rank; c->device = device;
  ncclResult_t r = n->CommInitRank(&c->comm, world_size, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return fail(MOLE_ERR_NCCL, "ncclCommInitRank -> %s", n->GetErrorString(r));
  }
  *out = c;
  return MOLE_OK;
}
extern "C" int mole_comm_destroy(mole_comm* c) {
  if (!c) return MOLE_OK;
  NcclApi* n = nccl_api();
  if (n) n->CommDestroy(c->comm);
  delete c;
  return MOLE_OK;
}
extern "C" int mole_all2all(mole_comm* c, const void* send, void* recv, int64_t bytes_per_peer,
                            int64_t peer_stride_bytes, void* stream) {
  MOLE_REQUIRE(c && send && recv && bytes_per_peer >= 0, "bad argument");
  MOLE_REQUIRE(peer_stride_bytes >= bytes_per_peer, "peer stride %lld < payload %lld",
               (long long)peer_stride_bytes, (long long)bytes_per_peer);
  NcclApi* n = nccl_api();
  if (!n) return fail(MOLE_ERR_NCCL, "libnccl.so.2 could not be loaded");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* s = static_cast<const char*>(send);
  char* r = static_cast<char*>(recv);
  MOLE_CUDA_OK(cudaMemcpyAsync(r + c->rank * peer_stride_bytes, s + c->rank * peer_stride_bytes,
                               (size_t)bytes_per_peer, cudaMemcpyDeviceToDevice, st));
  if (c->world == 1) return MOLE_OK;
  MOLE_NCCL_OK(n, n->GroupStart());
  for (int q = 0; q < c->world; ++q) {
    if (q == c->rank) continue;
    MOLE_NCCL_OK(n, n->Send(s + q * peer_stride_bytes, (size_t)bytes_per_peer, ncclInt8, q, c->comm, st));
    MOLE_NCCL_OK(n, n->Recv(r + q * peer_stride_bytes, (size_t)bytes_per_peer, ncclInt8, q, c->comm, st));
  }
  MOLE_NCCL_OK(n, n->GroupEnd());
  return MOLE_OK;
}

// ---- peer-visible buffers (push-style exchange) ------------------------------------------
// Plain cudaMalloc memory exported with the CUDA IPC handle: a peer process maps it and its
// kernels store rows straight into it over NVLink.  No multicast object is involved.
extern "C" int mole_peer_alloc(int64_t bytes, void** ptr) {
  MOLE_REQUIRE(ptr && bytes > 0, "bad argument");
  MOLE_CUDA_OK(cudaMalloc(ptr, (size_t)bytes));
  MOLE_CUDA_OK(cudaMemset(*ptr, 0, (size_t)bytes));
  return MOLE_OK;
}
extern "C" int mole_peer_free(void* ptr) {
  if (ptr) MOLE_CUDA_OK(cudaFree(ptr));
  return MOLE_OK;
}
extern "C" int mole_peer_export(void* ptr, uint8_t* handle64) {
  MOLE_REQUIRE(ptr && handle64, "bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  MOLE_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, 64);
  return MOLE_OK;
}
extern "C" int mole_peer_open(const uint8_t* handle64, void** ptr) {
  MOLE_REQUIRE(ptr && handle64, "bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  MOLE_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return MOLE_OK;
}
extern "C" int mole_peer_close(void* ptr) {
  if (ptr) MOLE_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return MOLE_OK;
}
// All ranks have reached this point of `stream` (and with it every kernel enqueued before): a
// 4-byte grouped send/recv with every peer.  `scratch` holds 8 * world bytes on the device.
extern "C" int mole_barrier(mole_comm* c, void* scratch, void* stream) {
  MOLE_REQUIRE(c && scratch, "bad argument");
  if (c->world == 1) return MOLE_OK;
  NcclApi* n = nccl_api();
  if (!n) return fail(MOLE_ERR_NCCL, "libnccl.so.2 could not be loaded");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* s = static_cast<char*>(scratch);
  MOLE_NCCL_OK(n, n->GroupStart());
  for (int q = 0; q < c->world; ++q) {
    if (q == c->rank) continue;
    MOLE_NCCL_OK(n, n->Send(s + 4 * q, 4, ncclInt8, q, c->comm, st));
    MOLE_NCCL_OK(n, n->Recv(s + 4 * (c->world + q), 4, ncclInt8, q, c->comm, st));
  }
  MOLE_NCCL_OK(n, n->GroupEnd());
  return MOLE_OK;
}

// The same barrier without NCCL: every rank stores the barrier's sequence number into its own
// entry of every peer's flag array (mapped peer memory, plain stores over NVLink) and waits until
// its own array shows the number from every peer.  One warp, one launch of a few microseconds
// instead of a grouped send/recv (~30 us at 8 ranks).  The wait is bounded: when it runs out the
// kernel records code 40 + the first missing rank in the fault word and returns, so a rank that
// never arrives costs its peers `limit_ns`, not a hung GPU.
struct PeerFlags { int32_t* flags[kMaxPeers]; };
__global__ void peer_barrier_kernel(const __grid_constant__ PeerFlags f, int world, int rank,
                                    int32_t seq, uint64_t limit_ns, int32_t* fault) {
  const int q = threadIdx.x;
  if (q >= world || q == rank) return;
  // what this GPU's earlier kernels stored into the peers' memory is ordered before the flag
  __threadfence_system();
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(f.flags[q] + rank), "r"(seq) : "memory");
  const int32_t* mine = f.flags[rank] + q;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t polls = 0;; ++polls) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - seq >= 0) return;                     // the peer has reached this barrier (or a later one)
    if ((polls & 0x3f) == 0x3f) {
      uint64_t t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > limit_ns) {
        atomicCAS(fault, 0, 40 + q);
        return;
      }
    }
  }
}

extern "C" int mole_peer_barrier(void* const* peer_flags, int32_t world, int32_t rank, int32_t seq,
                                 int64_t limit_ns, void* stream) {
  MOLE_REQUIRE(peer_flags != nullptr, "null flag table");
  MOLE_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world,
               "rank %d / world %d (at most %d ranks)", rank, world, kMaxPeers);
  MOLE_REQUIRE(limit_ns > 0, "the wait needs a limit");
  if (world == 1) return MOLE_OK;
  PeerFlags f{};
  for (int q = 0; q < world; ++q) {
    MOLE_REQUIRE(peer_flags[q] != nullptr, "null flag array of rank %d", q);
    f.flags[q] = static_cast<int32_t*>(peer_flags[q]);
  }
  int32_t* fault = device_fault_word();
  if (!fault) return fail(MOLE_ERR_CUDA, "fault word not allocated");
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, seq,
                                                                       (uint64_t)limit_ns, fault);
  MOLE_LAUNCH_OK();
  return MOLE_OK;
}

// ---- offloaded-expert slot pool -----------------------------------------------------
struct mole_pool {
  mole_ctx* ctx;
  int pool_size, M, F, dtype;
  size_t bytes[4];                 // per-expert bytes of W1, b1, W2, b2
  void* base[4];
  int virtual_offset, view_size;
  std::vector<std::pair<int, int>> stack;      // (moe_id, n)
  std::vector<cudaEvent_t> slot_event;         // last compute user of each absolute slot
  std::vector<char> slot_has;
  std::vector<cudaEvent_t> fetch_event;        // ticket ring
  int next_ticket;
  bool dry;                                    // no device: record the plan instead of running it
  std::vector<int32_t> log;                    // dry mode: {kind, a, b, c} per entry
};
static void pool_log(mole_pool* p, int kind, int a, int b, int c) {
  p->log.push_back(kind); p->log.push_back(a); p->log.push_back(b); p->log.push_back(c);
}
constexpr int kTickets = 256;

extern "C" int mole_pool_create(mole_ctx* ctx, int32_t pool_size, int32_t M, int32_t F,
                                int32_t dtype, mole_pool** out) {
  MOLE_REQUIRE(out != nullptr, "null argument");
  MOLE_REQUIRE(pool_size >= 1 && M > 0 && F > 0, "pool_size=%d M=%d F=%d", pool_size, M, F);
  MOLE_REQUIRE(dtype == MOLE_F32 || dtype == MOLE_BF16, "dtype %d", dtype);
  const size_t es = dtype == MOLE_F32 ? 4 : 2;
  mole_pool* p = new mole_pool();
  p->ctx = ctx; p->pool_size = pool_size; p->M = M; p->F = F; p->dtype = dtype;
  p->bytes[0] = (size_t)F * M * es; p->bytes[1] = (size_t)F * es;
  p->bytes[2] = (size_t)F * M * es; p->bytes[3] = (size_t)M * es;
  p->virtual_offset = 0; p->view_size = pool_size; p->next_ticket = 0;
  p->dry = ctx == nullptr;
  p->slot_has.assign(pool_size, 0);
  if (p->dry) {
    for (int i = 0; i < 4; ++i) p->base[i] = nullptr;
    *out = p;
    return MOLE_OK;
  }
  for (int i = 0; i < 4; ++i) {
    p->base[i] = nullptr;
    cudaError_t e = cudaMalloc(&p->base[i], p->bytes[i] * pool_size);
    if (e == cudaSuccess) e = cudaMemset(p->base[i], 0, p->bytes[i] * pool_size);
    if (e != cudaSuccess) {
      for (int j = 0; j <= i; ++j) if (p->base[j]) cudaFree(p->base[j]);
      delete p;
      return fail(MOLE_ERR_CUDA, "pool allocation failed: %s", cudaGetErrorString(e));
    }
  }
  p->slot_event.resize(pool_size);
  for (int i = 0; i < pool_size; ++i)
    MOLE_CUDA_OK(cudaEventCreateWithFlags(&p->slot_event[i], cudaEventDisableTiming));
  p->fetch_event.resize(kTickets);
  for (int i = 0; i < kTickets; ++i)
    MOLE_CUDA_OK(cudaEventCreateWithFlags(&p->fetch_event[i], cudaEventDisableTiming));
  *out = p;
  return MOLE_OK;
}
extern "C" int mole_pool_destroy(mole_pool* p) {
  if (!p) return MOLE_OK;
  for (int i = 0; i < 4; ++i) if (p->base[i]) cudaFree(p->base[i]);
  for (auto e : p->slot_event) cudaEventDestroy(e);
  for (auto e : p->fetch_event) cudaEventDestroy(e);
  delete p;
  return MOLE_OK;
}
extern "C" int mole_pool_base(mole_pool* p, int32_t p_id, void** base) {
  MOLE_REQUIRE(p && base && p_id >= 0 && p_id < 4, "bad argument");
  *base = p->base[p_id];
  return MOLE_OK;
}
extern "C" int mole_pool_view_size(mole_pool* p, int32_t* n) {
  MOLE_REQUIRE(p && n, "null argument");
  *n = p->view_size;
  return MOLE_OK;
}
extern "C" int mole_pool_clear_virtual(mole_pool* p) {
  MOLE_REQUIRE(p != nullptr, "pool is null");
  p->stack.clear();
  p->virtual_offset = 0;
  p->view_size = p->pool_size;
  return MOLE_OK;
}
extern "C" int mole_pool_prefetch(mole_pool* p, int32_t moe_id, int32_t n, int32_t* first_slot) {
  MOLE_REQUIRE(p && first_slot, "null argument");
  MOLE_REQUIRE(n >= 0, "n=%d", n);
  if (n > p->view_size)
    return fail(MOLE_ERR_STATE, "prefetch of %d experts exceeds the %d free slots", n, p->view_size);
  *first_slot = p->virtual_offset;
  if (n == 0) return MOLE_OK;
  if (!p->stack.empty() && p->stack.back().first == moe_id) p->stack.back().second += n;
  else p->stack.emplace_back(moe_id, n);
  p->virtual_offset += n;
  p->view_size -= n;
  return MOLE_OK;
}
extern "C" int mole_pool_pop_prefetched(mole_pool* p, int32_t moe_id, int32_t* n) {
  MOLE_REQUIRE(p && n, "null argument");
  *n = 0;
  if (!p->stack.empty() && p->stack.back().first == moe_id) {
    *n = p->stack.back().second;
    p->stack.pop_back();
    p->virtual_offset -= *n;
    p->view_size += *n;
  }
  return MOLE_OK;
}
extern "C" int mole_pool_abs_slot(mole_pool* p, int32_t view_slot, int32_t* abs_slot) {
  MOLE_REQUIRE(p && abs_slot, "null argument");
  MOLE_REQUIRE(view_slot >= 0 && view_slot + p->virtual_offset < p->pool_size,
               "view slot %d outside the visible pool", view_slot);
  *abs_slot = view_slot + p->virtual_offset;
  return MOLE_OK;
}
extern "C" int mole_pool_fetch(mole_pool* p, const void* const host_params[4], int64_t e0,
                               int32_t n, int32_t slot0, int32_t skip, int32_t absolute,
                               int32_t* ticket) {
  MOLE_REQUIRE(p && host_params && ticket, "null argument");
  MOLE_REQUIRE(n >= 0 && skip >= 0 && skip <= n && e0 >= 0, "n=%d skip=%d e0=%lld", n, skip, (long long)e0);
  const int a0 = absolute ? slot0 : slot0 + p->virtual_offset;
  if (slot0 < 0 || a0 + n > p->pool_size)
    return fail(MOLE_ERR_STATE, "slots [%d,%d) outside the pool of %d", a0, a0 + n, p->pool_size);
  if (p->dry) {
    for (int i = skip; i < n; ++i)
      if (p->slot_has[a0 + i]) pool_log(p, 2, a0 + i, 0, 0);
    if (n > skip) pool_log(p, 0, (int)(e0 + skip), a0 + skip, n - skip);
    *ticket = p->next_ticket;
    p->next_ticket = (p->next_ticket + 1) % kTickets;
    return MOLE_OK;
  }
  cudaStream_t tran = p->ctx->streams[1];
  for (int i = skip; i < n; ++i)
    if (p->slot_has[a0 + i]) MOLE_CUDA_OK(cudaStreamWaitEvent(tran, p->slot_event[a0 + i], 0));
  if (n > skip) {
    for (int k = 0; k < 4; ++k) {
      MOLE_REQUIRE(host_params[k] != nullptr, "host parameter %d is null", k);
      const char* src = static_cast<const char*>(host_params[k]) + (size_t)(e0 + skip) * p->bytes[k];
      char* dst = static_cast<char*>(p->base[k]) + (size_t)(a0 + skip) * p->bytes[k];
      MOLE_CUDA_OK(cudaMemcpyAsync(dst, src, p->bytes[k] * (size_t)(n - skip),
                                   cudaMemcpyHostToDevice, tran));
    }
  }
  *ticket = p->next_ticket;
  MOLE_CUDA_OK(cudaEventRecord(p->fetch_event[p->next_ticket], tran));
  p->next_ticket = (p->next_ticket + 1) % kTickets;
  return MOLE_OK;
}
extern "C" int mole_pool_wait_fetch(mole_pool* p, int32_t ticket, void* stream) {
  MOLE_REQUIRE(p && ticket >= 0 && ticket < kTickets, "bad ticket %d", ticket);
  if (p->dry) return MOLE_OK;
  MOLE_CUDA_OK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), p->fetch_event[ticket], 0));
  return MOLE_OK;
}
extern "C" int mole_pool_mark_used(mole_pool* p, int32_t slot0, int32_t n, void* stream) {
  MOLE_REQUIRE(p != nullptr, "pool is null");
  const int a0 = slot0 + p->virtual_offset;
  if (slot0 < 0 || n < 0 || a0 + n > p->pool_size)
    return fail(MOLE_ERR_STATE, "slots [%d,%d) outside the pool of %d", a0, a0 + n, p->pool_size);
  if (p->dry && n > 0) pool_log(p, 1, a0, n, 0);
  for (int i = 0; i < n; ++i) {
    if (!p->dry)
      MOLE_CUDA_OK(cudaEventRecord(p->slot_event[a0 + i], static_cast<cudaStream_t>(stream)));
    p->slot_has[a0 + i] = 1;
  }
  return MOLE_OK;
}
extern "C" int mole_pool_log(mole_pool* p, int32_t* out, int32_t capacity, int32_t* n_entries) {
  MOLE_REQUIRE(p && n_entries, "null argument");
  const int n = (int)(p->log.size() / 4);
  *n_entries = n;
  if (out)
    for (int i = 0; i < n * 4 && i < capacity * 4; ++i) out[i] = p->log[i];
  return MOLE_OK;
}
