// Device-side pieces of the tensor-parallel exchanges over peer memory (see tp_collectives.cu
// for the protocol): the table of peer mappings, system-scope loads and stores, the flag
// exchange, and a per-CTA maximum over ranks that other kernels can call in passing.
#pragma once

#include "common.cuh"

namespace xaxb {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxSlots = 1024;
// Waits on other GPUs get a longer limit than waits inside one GPU (ranks reach an exchange at
// different times: graph upload, host jitter; peer_wait_limit_ns, 10 s unless changed), and once
// any wait of this context has given up -- the status word is set -- later waits return at once,
// so a broken run drains quickly.
constexpr int kSiteTpSum = 41, kSiteTpMax = 42, kSiteTpSilu = 43, kSiteTpAttn = 44;

// Flag region of one exchange kind: flags[kTpMaxSlots][kTpMaxWorld] then epoch[kTpMaxSlots].
constexpr int64_t kTpSyncBytes = (int64_t)(kTpMaxSlots * kTpMaxWorld + kTpMaxSlots) * 4;

struct PeerTable {
  uint8_t* base[kTpMaxWorld];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// Raise this rank's flag for `slot` on every rank and wait until every rank has raised its
// flag here.  Called by all threads of the CTA; threads 0 .. world-1 do the work.  Returns the
// epoch of this exchange (the same in every thread).  `s_epoch` is one uint32 of shared memory.
__device__ __forceinline__ uint32_t tp_exchange_flags(const PeerTable& peers, int64_t sync_off, int rank, int world,
                                                      int slot, uint32_t* s_epoch, int* d_status, int site) {
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(peers.base[rank] + sync_off);
  uint32_t* my_epoch = my_flags + kTpMaxSlots * kTpMaxWorld + slot;
  if (threadIdx.x == 0) {
    const uint32_t e = *my_epoch + 1;
    *my_epoch = e;
    *s_epoch = e;
  }
  __syncthreads();  // also: every thread's earlier stores precede the release stores below
  const uint32_t epoch = *s_epoch;
  if ((int)threadIdx.x < world) {
    const int r = threadIdx.x;
    uint32_t* theirs = reinterpret_cast<uint32_t*>(peers.base[r] + sync_off) + slot * kTpMaxWorld + rank;
    st_release_sys(theirs, epoch);  // cumulative over the CTA's stores: they precede the barrier above
    const uint32_t* mine = my_flags + slot * kTpMaxWorld + r;
    if ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      const unsigned long long t0 = globaltimer_ns();
      const unsigned long long limit = peer_wait_limit_ns(d_status);
      while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
        if (*reinterpret_cast<volatile int*>(d_status) != 0) break;
        if (globaltimer_ns() - t0 > limit) {
          atomicCAS(d_status, 0, XAXB_DEVICE_TIMEOUT * 1000 + site);
          break;
        }
      }
    }
  }
  __syncthreads();
  return epoch;
}

// Inbox of the per-CTA maximum: uint64 [2][kTpMaxWorld][kTpMaxSlots], used in alternation by
// epoch parity.  An entry is (epoch << 32 | value): value and "it has arrived" travel in ONE 8-byte
// store, which is single-copy atomic, so the exchange needs no fence, no releasing store and no
// acquiring load -- each of those costs a few microseconds at system scope, and this exchange sits
// on the critical path of two kernels per transformer block.
constexpr int64_t kTpRowMaxInboxBytes = 2ll * kTpMaxWorld * kTpMaxSlots * 8;

// What a kernel needs to take the maximum of one 32-bit value per CTA over the ranks; world <= 1
// means "no exchange".  Passed by value.  sync_off: only the epoch counters of the flag region are used.
struct TpRowMax {
  PeerTable peers;
  int64_t inbox_off, sync_off;
  int rank, world;
};

// max over ranks of `mine` (compared as unsigned integers: the bit pattern of a non-negative
// amax, so NaN wins as it does in the quantiser) for CTA `slot`; the matching CTA of every rank
// must call it.  Thread r < world stores (epoch, value) into rank r's inbox and polls this rank's
// inbox until rank r's entry carries this epoch; the maximum is then shared through `s_tmp` (two
// uint32 of shared memory).  Called by all threads of the CTA.  An entry of epoch e is overwritten
// by epoch e + 2 at the earliest, which its writer reaches only after it has seen this rank's entry
// of epoch e + 1, i.e. after this CTA finished reading epoch e (stream order on this rank).
__device__ __forceinline__ uint32_t tp_cta_max_u32(const TpRowMax& tp, int slot, uint32_t mine, uint32_t* s_tmp,
                                                   int* d_status, int site) {
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(tp.peers.base[tp.rank] + tp.sync_off);
  uint32_t* my_epoch = my_flags + kTpMaxSlots * kTpMaxWorld + slot;
  if (threadIdx.x == 0) {
    const uint32_t e = *my_epoch + 1;
    *my_epoch = e;
    s_tmp[0] = e;
    s_tmp[1] = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_tmp[0];
  if ((int)threadIdx.x < tp.world) {
    const int r = threadIdx.x;
    const int64_t box = tp.inbox_off + (int64_t)(epoch & 1) * kTpMaxWorld * kTpMaxSlots * 8;
    unsigned long long* their_box =
        reinterpret_cast<unsigned long long*>(tp.peers.base[r] + box) + tp.rank * kTpMaxSlots + slot;
    const unsigned long long word = ((unsigned long long)epoch << 32) | mine;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(their_box), "l"(word) : "memory");
    const unsigned long long* my_box =
        reinterpret_cast<const unsigned long long*>(tp.peers.base[tp.rank] + box) + r * kTpMaxSlots + slot;
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(my_box) : "memory");
    if ((uint32_t)(w >> 32) != epoch) {
      const unsigned long long t0 = globaltimer_ns();
      const unsigned long long limit = peer_wait_limit_ns(d_status);
      for (;;) {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(my_box) : "memory");
        if ((uint32_t)(w >> 32) == epoch) break;
        __nanosleep(32);  // a hundred CTAs poll at once: leave the memory system to the stores they wait for
        if (*reinterpret_cast<volatile int*>(d_status) != 0) break;
        if (globaltimer_ns() - t0 > limit) {
          atomicCAS(d_status, 0, XAXB_DEVICE_TIMEOUT * 1000 + site);
          break;
        }
      }
    }
    if ((uint32_t)(w >> 32) == epoch) atomicMax(&s_tmp[1], (uint32_t)w);
  }
  __syncthreads();
  return s_tmp[1];
}

// Host side: checks the arguments of an entry point that takes a peer table and packs them.
inline int fill_tp_rowmax(TpRowMax& tp, void* const* peer_bases, int rank, int world, int64_t inbox_off,
                          int64_t sync_off, const char* what) {
  if (!peer_bases || world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world || (inbox_off & 15) ||
      (sync_off & 15) || inbox_off < 0 || sync_off < 0) {
    set_last_error("%s: needs 1 <= world <= %d, 0 <= rank < world, the table of peer mappings and aligned offsets",
                   what, kTpMaxWorld);
    return XAXB_BAD_ARGUMENT;
  }
  for (int r = 0; r < kTpMaxWorld; ++r) tp.peers.base[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (!peer_bases[r] || (reinterpret_cast<uintptr_t>(peer_bases[r]) & 15)) {
      set_last_error("%s: mapping of rank %d is null or not 16-byte aligned", what, r);
      return XAXB_BAD_ARGUMENT;
    }
    tp.peers.base[r] = static_cast<uint8_t*>(peer_bases[r]);
  }
  tp.inbox_off = inbox_off;
  tp.sync_off = sync_off;
  tp.rank = rank;
  tp.world = world;
  return XAXB_OK;
}

}  // namespace xaxb
