// Peer-memory communication context shared by the fused compute+collective kernels.
//
// Every rank of a tensor/expert-parallel group owns one "symmetric" buffer (same layout on every rank),
// allocated with cudaMalloc and mapped into the peers through CUDA IPC. Kernels push data into peers with
// plain stores over NVLink (P2P), publish it with a system-scope release store of a sequence number into
// the peer's flag word, and wait on their *local* flag words with acquire loads. Every wait is bounded.
// No TMA load with cluster multicast ever touches this memory.
//
// Layout of a symmetric buffer (offsets identical on all ranks):
//   flags : [2 parity][kMaxRanks src][kMaxFlags] u32   sequence numbers
//   data  : [2 parity][kMaxRanks src][slot_bytes]      staging area written by `src`
//   out   : [out_bytes]                                gather target (final layout)
//   lam   : [2 parity][kMaxRanks src][lam_bytes]       one-shot all-reduce words without tags (see below)
// plus two local words (not touched by peers): seq (calls completed) and done (CTA exit counter).
#pragma once
#include <stdint.h>

#include "ptx.cuh"

namespace eredu {

constexpr int kMaxRanks = 8;
constexpr int kMaxFlags = 8192;

struct PeerComm {
  uint8_t* base[kMaxRanks];  // peer r's symmetric buffer as mapped in this process (base[rank] = own)
  int rank;
  int size;
  long long flags_off;   // byte offsets inside a symmetric buffer
  long long data_off;
  long long out_off;
  long long slot_bytes;  // bytes per (parity, src) staging slot
  long long lam_off;     // sentinel-initialised region of the tag-free one-shot all-reduce
  long long lam_bytes;   // bytes per (parity, src) slot of that region
  unsigned int* seq;     // local
  unsigned int* done;    // local
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ unsigned int* peer_flag(const PeerComm& c, int peer, int parity, int src, int idx) {
  return reinterpret_cast<unsigned int*>(c.base[peer] + c.flags_off) + (static_cast<size_t>(parity) * kMaxRanks + src) * kMaxFlags + idx;
}
__device__ __forceinline__ uint8_t* peer_slot(const PeerComm& c, int peer, int parity, int src) {
  return c.base[peer] + c.data_off + (static_cast<size_t>(parity) * kMaxRanks + src) * c.slot_bytes;
}

// Tag-free one-shot words ("Lamport" style): the region starts as all-ones words; a writer never sends that pattern
// (a bf16 pair of two all-ones NaNs is replaced by canonical NaNs), so a 4-byte word is valid as soon as it differs
// from the pattern - the whole word is payload. The single reader of a word writes the pattern back right after it
// has read the value. The slot of that parity is written again two calls later; a peer can only be two calls ahead
// after it has consumed this rank's words of the call in between, which this rank sends from a later kernel, so the
// write-back always lands first.
constexpr uint32_t kLamportEmpty = 0xFFFFFFFFu;
__device__ __forceinline__ uint8_t* lamport_slot(const PeerComm& c, int peer, int parity, int src) {
  return c.base[peer] + c.lam_off + (static_cast<size_t>(parity) * kMaxRanks + src) * c.lam_bytes;
}
__device__ __forceinline__ uint32_t lamport_payload(uint32_t v) { return v == kLamportEmpty ? 0x7FFF7FFFu : v; }

// Bounded wait until the local flag written by `src` reaches `want`. Sequence numbers only grow.
__device__ __forceinline__ bool wait_flag(const PeerComm& c, int parity, int src, int idx, unsigned int want, int* status) {
  const unsigned int* f = peer_flag(c, c.rank, parity, src, idx);
  if (static_cast<int>(ld_acquire_sys_u32(f) - want) >= 0) return true;
  const long long t0 = clock64();
  // poll with relaxed loads, acquire once at the end
  while (static_cast<int>(ld_relaxed_sys_u32(f) - want) < 0) {
    if (clock64() - t0 > kWaitCycleLimit) {
      report_status(status, kStatusPeerFlagTimeout);
      return false;
    }
  }
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  return true;
}

// Called by one thread per CTA after the CTA's last use of `seq`: the last CTA of the grid advances it.
__device__ __forceinline__ void finish_call(const PeerComm& c, unsigned int seq, unsigned int total_ctas) {
  __threadfence();
  if (atomicAdd(c.done, 1u) == total_ctas - 1) {
    *c.done = 0u;
    __threadfence();
    *c.seq = seq + 1u;
  }
}

}  // namespace eredu
