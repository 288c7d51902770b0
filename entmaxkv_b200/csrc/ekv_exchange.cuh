// Peer exchange for the sequence-sharded decode step: tiny all-reduces done by the
// consuming kernel itself over NVLink peer memory instead of by a collective library.
//
// Every rank owns one buffer ("inbox") that all peers have mapped.  A value travels as one
// naturally aligned 64-bit word {epoch : value bits}; a 64-bit scalar store is a single
// copy, so the receiver sees either the old word or the complete new one and needs no fence
// and no separate flag.  An exchange of n values on slot s:
//   1. the sender stores word i of its partials into region (s, parity, own rank) of every
//      PEER's inbox (plain peer stores; its own values never leave its registers),
//   2. the receiver, for every value it consumes, polls - with an iteration budget - the
//      words of the other ranks in its OWN inbox until they carry the current epoch (local
//      memory reads only), and combines the world's values in rank order, so every rank
//      computes bit-identical results.
// Nothing couples the threads of an exchange, so any grid works as long as the same thread
// layout is used by every rank.  The epoch is ONE number per slot and launch: every block reads
// the slot's counter when it starts, and the block that draws the launch's last ticket advances
// it - after every block has read it - so the k-th exchange on a slot carries epoch k on every
// rank whatever grids the earlier exchanges on that slot used, and a word left behind by an
// earlier exchange can never pass for the current one.  Consequently the launches that use one
// slot must be ordered (one stream, or explicit dependencies): two of them in flight at once
// would draw tickets from the same counter.
// Regions are double-buffered by epoch parity: a rank can run at most one exchange ahead of a
// peer on a slot, because the next exchange on that slot needs the peer's contribution,
// which the peer sends only after it has consumed the previous one.
//
// No multicast loads and no unbounded waits: when a thread's budget runs out it sets
// EKV_STATUS_PEER_TIMEOUT in the caller's status word, stops waiting for the rest of the
// exchange and finishes on whatever the words hold (in-bounds local memory), so the kernel
// returns and the context stays usable.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/entmaxkv_b200.h"

namespace ekv {

constexpr int kXchMaxRanks = EKV_EXCHANGE_MAX_RANKS;
constexpr int kXchFusedSlots = 4;     // slots 0..3: the four reductions of the fused sharded step
constexpr int kXchSlots = 8;          // slots 4..7: ekv_exchange_allreduce (its slot argument + 4)
constexpr int kXchThreads = 1024;
constexpr int kXchMaxBlocks = 4096;   // largest grid of an exchange kernel

// What a kernel needs of an exchange object (passed by value).
struct XchDev {
  unsigned long long* inbox[kXchMaxRanks];   // rank r's inbox (peer mapping; [rank] is local)
  unsigned* epochs;                          // local: [slot] {exchanges completed, tickets drawn by the running launch}
  int rank, world;
  int max_floats;                            // words per region
  unsigned spin_limit;                       // polling iterations a thread may spend per exchange
};

__device__ __forceinline__ size_t xch_region(const XchDev& x, int slot, unsigned parity, int src) {
  return ((size_t)(slot * 2 + parity) * kXchMaxRanks + src) * (size_t)x.max_floats;
}

__device__ __forceinline__ void st_word(unsigned long long* p, unsigned long long v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// One exchange as seen by one thread.
struct Xch {
  const XchDev* x;
  size_t off;          // word offset of region (slot, parity, rank 0); rank r's region is r * max_floats further
  unsigned epoch;
  unsigned budget;
  int* status;

  // Deliver this rank's value i to every peer.
  __device__ __forceinline__ void send(int i, float v) const {
    const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    for (int k = 1; k < x->world; ++k) {
      const int r = (x->rank + k) % x->world;
      st_word(x->inbox[r] + off + (size_t)x->rank * x->max_floats + i, w);
    }
  }

  // Rank r's value i (r != own rank); polls the local inbox until the word carries this epoch.
  __device__ __forceinline__ float wait(int r, int i) {
    const unsigned long long* p = x->inbox[x->rank] + off + (size_t)r * x->max_floats + i;
    unsigned long long w = ld_word(p);
    while ((unsigned)(w >> 32) != epoch) {
      if (budget == 0) {
        atomicOr(status, EKV_STATUS_PEER_TIMEOUT);
        break;
      }
      --budget;
      __nanosleep(32);
      w = ld_word(p);
    }
    return __uint_as_float((unsigned)w);
  }

  // Combine value i over the world in rank order; `mine` is this rank's own contribution.
  __device__ __forceinline__ float sum(int i, float mine) {
    float s = 0.f;
    for (int r = 0; r < x->world; ++r) {
      const float v = r == x->rank ? mine : wait(r, i);
      s = r == 0 ? v : s + v;
    }
    return s;
  }
  __device__ __forceinline__ float max(int i, float mine) {
    float s = 0.f;
    for (int r = 0; r < x->world; ++r) {
      const float v = r == x->rank ? mine : wait(r, i);
      s = r == 0 ? v : fmaxf(s, v);
    }
    return s;
  }
};

// Start an exchange on `slot`: block-collective (contains a __syncthreads); every block of the
// grid calls it exactly once per launch, before any early exit, and every rank launches the
// same grid.
__device__ __forceinline__ Xch xch_begin(const XchDev& x, int slot, int* status) {
  __shared__ unsigned s_epoch;
  if (threadIdx.x == 0) {
    unsigned* ctr = x.epochs + slot * 2;
    unsigned done;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(done) : "l"(ctr) : "memory");
    __threadfence();                                   // the counter is read before the ticket is drawn
    const unsigned n_blocks = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(ctr + 1, 1u) == n_blocks - 1u) {     // every block of this launch has read the counter
      ctr[1] = 0u;
      __threadfence();
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(ctr), "r"(done + 1u) : "memory");
    }
    s_epoch = done + 1u;
  }
  __syncthreads();
  Xch e;
  e.x = &x;
  e.epoch = s_epoch;
  e.budget = x.spin_limit;
  e.status = status;
  e.off = xch_region(x, slot, s_epoch & 1u, 0);
  return e;
}

// Host side (ekv_exchange.cu): the device view of an exchange object, or false if it is
// not connected yet.
bool xch_device_view(const ekv_exchange* x, XchDev* out);

}  // namespace ekv
