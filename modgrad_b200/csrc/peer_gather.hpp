// All-gather of small slices between the GPUs of one box by direct peer stores over NVLink:
// the latency-bound alternative to an NCCL all-gather inside the row-sharded decode loop.
//
// Every rank owns one `arena` (a cudaMalloc allocation mapped into the other processes with CUDA
// IPC).  All ranks lay their arenas out identically: a block of flags, then the gathered
// buffers.  A gather is ONE kernel per rank: it copies the rank's slice of a buffer into the
// same place of every peer's arena with plain stores, fences, publishes a per-(site, source)
// epoch flag on every peer, and waits — with a bounded spin — until the flags of all peers have
// reached the same epoch.  The kernels of different ranks run on different GPUs, so the wait
// never depends on another launch of the same GPU.
//
// Ordering contract for the caller: consecutive gathers must use different buffers (a rank can
// run at most one gather ahead of a peer, so it may already be storing gather k+1 while the
// peer still reads the result of gather k).  `site` names the flag set and the epoch counter;
// every rank must issue the gathers of a site in the same order.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "peer_sync.cuh"

namespace mgpeer {

constexpr int kMaxRanks = 8;
constexpr int kMaxSites = 8;
constexpr size_t kFlagBytes = 4096;  // head of every arena: flag[site][source rank], 64 bytes apart

struct Exchange {
    int rank = 0, world = 1;
    unsigned char* base[kMaxRanks] = {};  // base[r]: rank r's arena as mapped in this process
    unsigned* ctl = nullptr;              // local control words: epochs, tickets, error (see .cu)
    size_t bytes = 0;                     // size of the arena (the same on every rank)
    unsigned spin_limit = kSyncSpinLimit; // polls before a bounded wait gives up
};
constexpr size_t kCtlWords = 2 * kMaxSites + 1;
static_assert(kMaxRanks == kSyncMaxRanks && kMaxSites == kSyncMaxSites && kFlagBytes == kSyncFlagBytes, "one layout");

// The device-side view of exchange `site` (what a fused kernel is given).
PeerSync make_sync(const Exchange& ex, int site);

// Copies bytes [offset + my_off, offset + my_off + my_bytes) of the local arena to every peer and
// completes the exchange of `site`.  offset, my_off and my_bytes are multiples of 4.
cudaError_t launch_gather(const Exchange& ex, int site, size_t offset, size_t my_off, size_t my_bytes,
                          cudaStream_t stream);
// 0, or 1 + the site whose wait ran out (the gathered data of that call is incomplete).
cudaError_t read_error(const Exchange& ex, int* site_plus_one);

}  // namespace mgpeer
