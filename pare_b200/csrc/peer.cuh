// Row-parallel sum over tensor-parallel ranks, fused into the epilogue of the W4A16 decode kernels.
//
// A row-parallel linear (the o and down projections of a tensor-parallel block) produces, on every rank, a
// partial output over its slice of the input columns; the ranks' partials have to be added.  Instead of a
// separate all-reduce launch, the thread that finishes an output element stores its fp32 partial into that
// element's slot of EVERY rank's exchange buffer (plain 8-byte peer stores over NVLink: {value, epoch}, so
// each element carries its own validity mark and there is neither a fence nor a flag), then reads the
// `world` slots of the element from its own GPU's buffer, spinning (bounded) until each shows the epoch of
// this call, adds them in rank order and writes the final value.  Every rank computes every element from
// the same fp32 partials in the same order: identical bits everywhere, one rounding to the output dtype.
// In the persistent kernel this runs in the epilogue warps while the consumer warps stream the next rows.
//
// Exchange buffer (pare_peer_buffer_create): [0, 4096) header -- int words: 0..15 epochs of the stand-alone
// all-reduce's CTAs, 16 status, 32 epoch of the fused exchange, 33 its exit counter; the data area behind
// the header is split in two halves, the first for the stand-alone all-reduce, the second for the fused
// exchange: [2 parities][world ranks][slot].  The epoch of a call is (word 32) + 1; the last of the call's
// exchanging units to finish advances the word.  Slots are double-buffered by the epoch's parity: a rank
// needs every peer's data of call n to finish call n, so it can be at most one call ahead of any peer and
// never overwrites a slot that is still being read.
// No multicast of any kind: plain stores to peer pointers, plain volatile loads from own memory.
#pragma once

#include "common.cuh"

namespace pare {

constexpr int kPeerMaxRanks = 8;
constexpr size_t kPeerHeaderBytes = 4096;
constexpr int kPeerStatusWord = 16;
constexpr int kPeerFusedEpochWord = 32;
constexpr int kPeerFusedExitWord = 33;
constexpr uint32_t kPeerFusedSpinLimit = 1u << 24;

// byte offset of the fused exchange's half of the data area
__host__ __device__ inline size_t peer_fused_offset(size_t buffer_bytes) {
  return kPeerHeaderBytes + (((buffer_bytes - kPeerHeaderBytes) / 2) & ~(size_t)255);
}

struct PeerCtx {
  unsigned char* buf[kPeerMaxRanks];   // buf[0] == nullptr: no exchange
  int rank, world;
  size_t data_off;     // peer_fused_offset(buffer_bytes)
  size_t slot_bytes;   // bytes per (parity, rank) slot
};

__host__ __device__ __forceinline__ bool peer_on(const PeerCtx& pc) { return pc.buf[0] != nullptr; }

// epoch of this call (read after the dependency wait: the previous call has advanced the word by then)
__device__ __forceinline__ uint32_t peer_epoch(const PeerCtx& pc) {
  const volatile int* hdr = reinterpret_cast<const volatile int*>(pc.buf[pc.rank]);
  return (uint32_t)hdr[kPeerFusedEpochWord] + 1u;
}

// this rank's fp32 partial of element idx into every rank's buffer
__device__ __forceinline__ void peer_send(const PeerCtx& pc, uint32_t e, size_t idx, float v) {
  const size_t off = pc.data_off + ((size_t)((e & 1u) * pc.world + pc.rank)) * pc.slot_bytes + idx * 8;
  for (int q = 0; q < pc.world; ++q)   // one 8-byte store: value and mark arrive together
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(pc.buf[q] + off), "r"(__float_as_uint(v)), "r"(e) : "memory");
}

__device__ __forceinline__ uint2 peer_ld_unit(const void* p) {
  uint2 u;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(u.x), "=r"(u.y) : "l"(p) : "memory");
  return u;
}

// sum of the ranks' partials of element idx, in rank order, as they arrive (bounded wait)
__device__ __forceinline__ float peer_recv(const PeerCtx& pc, uint32_t e, size_t idx, bool& timed_out) {
  const unsigned char* base = pc.buf[pc.rank] + pc.data_off + ((size_t)((e & 1u) * pc.world)) * pc.slot_bytes + idx * 8;
  float acc = 0.f;
  for (int q = 0; q < pc.world; ++q) {
    const unsigned char* src = base + (size_t)q * pc.slot_bytes;
    uint2 u = peer_ld_unit(src);
    uint32_t i = 0;
    while (u.y != e && !timed_out) {
      if (++i >= kPeerFusedSpinLimit) timed_out = true;
      u = peer_ld_unit(src);
    }
    acc += __uint_as_float(u.x);
  }
  return acc;
}

// One exchanging unit (a warp or a CTA: `total` of them per call) is done; the last one advances the epoch word.
// Called by one thread after all of the unit's receives.
__device__ __forceinline__ void peer_unit_done(const PeerCtx& pc, uint32_t e, int total, bool timed_out) {
  int* hdr = reinterpret_cast<int*>(pc.buf[pc.rank]);
  if (timed_out) atomicExch(hdr + kPeerStatusWord, PARE_ERR_TIMEOUT);
  __threadfence();
  if (atomicAdd(hdr + kPeerFusedExitWord, 1) == total - 1) {
    hdr[kPeerFusedExitWord] = 0;
    __threadfence();
    *reinterpret_cast<volatile int*>(hdr + kPeerFusedEpochWord) = (int)e;
  }
}

}  // namespace pare
