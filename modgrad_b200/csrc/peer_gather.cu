// See peer_gather.hpp.
#include <stdint.h>

#include "launch_common.cuh"
#include "peer_gather.hpp"

namespace mgpeer {
namespace {

constexpr int kThreads = 256;

struct Args {
    PeerSync ps;
    unsigned long long begin, bytes;  // slice inside the arena
};

__global__ void __launch_bounds__(kThreads) peer_gather_kernel(const Args a) {
    mg::pdl_prologue();  // the slice is written by the kernel launched just before this one
    const unsigned char* src = a.ps.base[a.ps.rank] + a.begin;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
    if (((a.begin | a.bytes) & 15u) == 0) {
        const size_t n = a.bytes / 16;
        for (size_t i = tid; i < n; i += nthr) {
            const uint4 v = reinterpret_cast<const uint4*>(src)[i];
            for (int p = 0; p < a.ps.world; ++p)
                if (p != a.ps.rank) reinterpret_cast<uint4*>(a.ps.base[p] + a.begin)[i] = v;
        }
    } else {
        const size_t n = a.bytes / 4;
        for (size_t i = tid; i < n; i += nthr) {
            const uint32_t v = reinterpret_cast<const uint32_t*>(src)[i];
            for (int p = 0; p < a.ps.world; ++p)
                if (p != a.ps.rank) reinterpret_cast<uint32_t*>(a.ps.base[p] + a.begin)[i] = v;
        }
    }
    peer_finish(a.ps);
}

}  // namespace

cudaError_t launch_gather(const Exchange& ex, int site, size_t offset, size_t my_off, size_t my_bytes,
                          cudaStream_t stream) {
    if (ex.world < 2 || ex.world > kMaxRanks || site < 0 || site >= kMaxSites || !ex.ctl) return cudaErrorInvalidValue;
    if (((offset | my_off | my_bytes) & 3u) != 0 || offset < kFlagBytes) return cudaErrorInvalidValue;
    if (offset + my_off > ex.bytes || my_bytes > ex.bytes - (offset + my_off)) return cudaErrorInvalidValue;
    Args a;
    a.ps = make_sync(ex, site);
    a.begin = offset + my_off;
    a.bytes = my_bytes;
    size_t ctas = (my_bytes + 8191) / 8192;
    if (ctas < 1) ctas = 1;
    if (ctas > 8) ctas = 8;
    return mg::launch_pdl(peer_gather_kernel, dim3((unsigned)ctas), dim3(kThreads), 0, stream, a);
}

PeerSync make_sync(const Exchange& ex, int site) {
    PeerSync ps;
    for (int r = 0; r < kSyncMaxRanks; ++r) ps.base[r] = r < ex.world ? ex.base[r] : nullptr;
    ps.ctl = ex.ctl;
    ps.arena_bytes = ex.bytes;
    ps.stamp_slots = nullptr; ps.epoch_dev = nullptr; ps.epoch_mul = 0; ps.epoch_add = 0; ps.stamp_index0 = 0;
    ps.rank = ex.rank; ps.world = ex.world; ps.site = site;
    ps.spin_limit = ex.spin_limit;
    return ps;
}

namespace {
thread_local PeerSync g_next = {};
thread_local StampIn g_next_in = {};
}
void set_next_stamp_in(const StampIn& in) { g_next_in = in; }
StampIn take_next_stamp_in() {
    const StampIn in = g_next_in;
    g_next_in = StampIn{};
    return in;
}
void set_next_peer_sync(const PeerSync& ps) { g_next = ps; }
PeerSync take_next_peer_sync() {
    const PeerSync ps = g_next;
    g_next = PeerSync{};
    return ps;
}

cudaError_t read_error(const Exchange& ex, int* site_plus_one) {
    unsigned v = 0;
    const cudaError_t e = cudaMemcpy(&v, ex.ctl + 2 * kMaxSites, sizeof v, cudaMemcpyDeviceToHost);
    if (site_plus_one) *site_plus_one = (int)v;
    return e;
}

}  // namespace mgpeer

// ---- C ABI: an exchange an engine outside this library can own ------------------------------
struct mg_peer_exchange {
    mgpeer::Exchange ex;
    size_t bytes = 0;
    void* opened[mgpeer::kMaxRanks] = {};
};

extern "C" {

// Allocates this rank's arena (`bytes`, zeroed; the first mg_peer_arena_offset() bytes hold the
// flags) and returns its CUDA IPC handle (64 bytes) for the other ranks.
int mg_peer_exchange_create(size_t bytes, int rank, int world, void* ipc_handle_out64, mg_peer_exchange** out) {
    if (!out || !ipc_handle_out64 || world < 2 || world > mgpeer::kMaxRanks || rank < 0 || rank >= world ||
        bytes <= mgpeer::kFlagBytes)
        return (int)cudaErrorInvalidValue;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    mg_peer_exchange* x = new mg_peer_exchange();
    x->ex.rank = rank; x->ex.world = world; x->ex.bytes = bytes; x->bytes = bytes;
    void* arena = nullptr;
    cudaError_t e = cudaMalloc(&arena, bytes);
    if (e == cudaSuccess) e = cudaMemset(arena, 0, bytes);
    void* ctl = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&ctl, mgpeer::kCtlWords * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctl, 0, mgpeer::kCtlWords * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle_out64), arena);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(arena); cudaFree(ctl);
        delete x;
        return (int)e;
    }
    x->ex.base[rank] = static_cast<unsigned char*>(arena);
    x->ex.ctl = static_cast<unsigned*>(ctl);
    *out = x;
    return 0;
}
// handles: world x 64 bytes, entry r = the handle rank r got from mg_peer_exchange_create (all
// ranks must have created their arenas before any rank calls this, e.g. after a host barrier).
int mg_peer_exchange_open(mg_peer_exchange* x, const void* handles) {
    if (!x || !handles) return (int)cudaErrorInvalidValue;
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(handles);
    for (int r = 0; r < x->ex.world; ++r) {
        if (r == x->ex.rank) continue;
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return (int)e;
        x->opened[r] = p;
        x->ex.base[r] = static_cast<unsigned char*>(p);
    }
    return 0;
}
void* mg_peer_arena(mg_peer_exchange* x) { return x ? x->ex.base[x->ex.rank] : nullptr; }
size_t mg_peer_arena_offset(void) { return mgpeer::kFlagBytes; }
// The next launch, from this host thread, of a kernel that supports it (launch_matvec_q4k* with y
// inside the arena, mg_swiglu_limbs_on_stream, mg_sdpa_decode_f16kv_on_stream) also stores its
// output into every peer's arena and ends with the exchange of `site` (0..7).
int mg_peer_fuse_next(mg_peer_exchange* x, int site) {
    if (!x || site < 0 || site >= mgpeer::kMaxSites) return (int)cudaErrorInvalidValue;
    for (int r = 0; r < x->ex.world; ++r)
        if (!x->ex.base[r]) return (int)cudaErrorInvalidValue;  // not opened yet
    mgpeer::set_next_peer_sync(mgpeer::make_sync(x->ex, site));
    return 0;
}
// Stand-alone gather of bytes [offset + my_off, offset + my_off + my_bytes) of the arena.
int mg_peer_gather_on_stream(mg_peer_exchange* x, int site, size_t offset, size_t my_off, size_t my_bytes,
                             void* stream) {
    if (!x) return (int)cudaErrorInvalidValue;
    return (int)mgpeer::launch_gather(x->ex, site, offset, my_off, my_bytes, (cudaStream_t)stream);
}
// Polls a bounded wait of this exchange makes before it gives up and sets the error word (default
// 1 << 22, a few seconds; a test that lets a wait run out on purpose lowers it).  Applies to
// launches armed afterwards.
int mg_peer_exchange_set_spin_limit(mg_peer_exchange* x, unsigned polls) {
    if (!x || polls == 0) return (int)cudaErrorInvalidValue;
    x->ex.spin_limit = polls;
    return 0;
}
// 0, or 1 + the site whose bounded wait ran out since creation; negative = -(CUDA error).
int mg_peer_exchange_status(mg_peer_exchange* x) {
    if (!x) return -(int)cudaErrorInvalidValue;
    int site = 0;
    const cudaError_t e = mgpeer::read_error(x->ex, &site);
    return e == cudaSuccess ? site : -(int)e;
}
void mg_peer_exchange_destroy(mg_peer_exchange* x) {
    if (!x) return;
    for (int r = 0; r < mgpeer::kMaxRanks; ++r)
        if (x->opened[r]) cudaIpcCloseMemHandle(x->opened[r]);
    cudaFree(x->ex.base[x->ex.rank]);
    cudaFree(x->ex.ctl);
    delete x;
}

}  // extern "C"
