// Host side of the peer exchange: the inbox allocation, its export to / import from the
// other ranks' processes, and a plain all-reduce kernel built on the word protocol of
// ekv_exchange.cuh.  The fused "exchange + epilogue" kernels of the sharded step live next
// to the arithmetic they finish (ekv_gaussian.cu, ekv_decode.cu).
#include <new>

#include "ekv_common.cuh"
#include "ekv_exchange.cuh"

struct ekv_exchange {
  int rank = 0, world = 0, max_floats = 0, device = 0;
  unsigned spin_limit = 1u << 21;          // polls per thread and exchange (each a load + 32 ns sleep): about a second
  char* base = nullptr;                    // local allocation: inbox words | epoch counters
  size_t bytes = 0;
  char* peer_base[EKV_EXCHANGE_MAX_RANKS] = {};
  bool opened_ipc[EKV_EXCHANGE_MAX_RANKS] = {};
  bool connected = false;
};

namespace ekv {

static size_t xch_data_bytes(int max_floats) {
  return (size_t)kXchSlots * 2 * kXchMaxRanks * (size_t)max_floats * sizeof(unsigned long long);
}
static size_t xch_epoch_bytes() { return 256; }   // kXchSlots x {epoch, tickets}, padded

bool xch_device_view(const ekv_exchange* x, XchDev* out) {
  if (!x || !x->connected) return false;
  for (int r = 0; r < kXchMaxRanks; ++r)
    out->inbox[r] = reinterpret_cast<unsigned long long*>(x->peer_base[r < x->world ? r : x->rank]);
  out->epochs = reinterpret_cast<unsigned*>(x->base + xch_data_bytes(x->max_floats));
  out->rank = x->rank;
  out->world = x->world;
  out->max_floats = x->max_floats;
  out->spin_limit = x->spin_limit;
  return true;
}

// dst[i] = reduce over ranks of src[i]; any grid of kXchThreads-thread blocks.
__global__ void __launch_bounds__(kXchThreads) xch_allreduce_kernel(const XchDev x, int slot,
                                                                    const float* __restrict__ src, int n, int op,
                                                                    float* __restrict__ dst, int* status) {
  Xch e = xch_begin(x, slot, status);
  const int first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
  for (int i = first; i < n; i += stride) e.send(i, src[i]);
  for (int i = first; i < n; i += stride) dst[i] = op == EKV_XCH_MAX ? e.max(i, src[i]) : e.sum(i, src[i]);
}

}  // namespace ekv

extern "C" int ekv_exchange_create(int32_t rank, int32_t world, int32_t max_floats, ekv_exchange** out) {
  using namespace ekv;
  if (!out || world < 1 || world > kXchMaxRanks || rank < 0 || rank >= world || max_floats < 4 ||
      max_floats % 4 || max_floats > kXchMaxBlocks * kXchThreads)
    return EKV_ERR_ARG;
  ekv_exchange* x = new (std::nothrow) ekv_exchange;
  if (!x) return EKV_ERR_ARG;
  x->rank = rank;
  x->world = world;
  x->max_floats = max_floats;
  cudaError_t e = cudaGetDevice(&x->device);
  x->bytes = xch_data_bytes(max_floats) + xch_epoch_bytes();
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&x->base), x->bytes);
  if (e == cudaSuccess) e = cudaMemset(x->base, 0, x->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (x->base) cudaFree(x->base);
    delete x;
    return (int)e;
  }
  x->peer_base[rank] = x->base;
  if (world == 1) x->connected = true;
  *out = x;
  return 0;
}

extern "C" int ekv_exchange_handle(const ekv_exchange* x, void* handle_out) {
  if (!x || !handle_out) return EKV_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == EKV_EXCHANGE_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, x->base);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

extern "C" int ekv_exchange_connect(ekv_exchange* x, const void* all_handles) {
  if (!x || !all_handles || x->connected) return EKV_ERR_ARG;
  const char* hs = static_cast<const char*>(all_handles);
  for (int r = 0; r < x->world; ++r) {
    if (r == x->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, hs + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    x->peer_base[r] = static_cast<char*>(p);
    x->opened_ipc[r] = true;
  }
  x->connected = true;
  return 0;
}

extern "C" void* ekv_exchange_base(const ekv_exchange* x) { return x ? x->base : nullptr; }

extern "C" int ekv_exchange_connect_pointers(ekv_exchange* x, void* const* bases) {
  if (!x || !bases || x->connected) return EKV_ERR_ARG;
  for (int r = 0; r < x->world; ++r) {
    if (r == x->rank) continue;
    if (!bases[r]) return EKV_ERR_ARG;
    x->peer_base[r] = static_cast<char*>(bases[r]);
  }
  x->connected = true;
  return 0;
}

extern "C" int ekv_exchange_set_spin_limit(ekv_exchange* x, uint32_t iterations) {
  if (!x || iterations == 0) return EKV_ERR_ARG;
  x->spin_limit = iterations;
  return 0;
}

extern "C" int ekv_exchange_destroy(ekv_exchange* x) {
  if (!x) return EKV_ERR_ARG;
  cudaError_t first = cudaSuccess;
  for (int r = 0; r < x->world; ++r)
    if (x->opened_ipc[r]) {
      cudaError_t e = cudaIpcCloseMemHandle(x->peer_base[r]);
      if (first == cudaSuccess) first = e;
    }
  cudaError_t e = cudaFree(x->base);
  if (first == cudaSuccess) first = e;
  delete x;
  return (int)first;
}

extern "C" int ekv_exchange_allreduce(ekv_exchange* x, int32_t slot, const float* src, float* dst, int32_t n,
                                      int32_t op, int32_t* status, void* stream) {
  using namespace ekv;
  XchDev d;
  if (!xch_device_view(x, &d) || !src || !dst || !status || n <= 0 || n > x->max_floats || slot < 0 ||
      slot >= kXchSlots - kXchFusedSlots || (op != EKV_XCH_SUM && op != EKV_XCH_MAX))
    return EKV_ERR_ARG;
  slot += kXchFusedSlots;   // slots of its own: the fused step's kernels keep theirs to themselves
  const int blocks = (n + kXchThreads - 1) / kXchThreads;     // <= max_floats / 1024, far below kXchMaxBlocks
  xch_allreduce_kernel<<<blocks, kXchThreads, 0, as_stream(stream)>>>(d, slot, src, n, op, dst, status);
  return launch_status();
}
