// Device side of the peer-store exchange (peer_gather.hpp): what a kernel needs to finish its
// own output with an all-gather — store every result word into the peers' arenas as well, then
// call peer_finish() once from all threads of every CTA.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgpeer {

constexpr int kSyncMaxRanks = 8;
constexpr int kSyncMaxSites = 8;
constexpr unsigned kSyncSpinLimit = 1u << 22;  // a few seconds of polling (covers host-side skew between the ranks), then give up

// world <= 1: no exchange (every helper below is then a no-op).
struct PeerSync {
    unsigned char* base[kSyncMaxRanks];  // base[r]: rank r's arena as mapped in this process
    unsigned* ctl;                       // local: [site] epoch, [kSyncMaxSites + site] ticket, [2*kSyncMaxSites] error
    unsigned long long arena_bytes;      // size of every rank's arena (all ranks lay theirs out identically)
    int rank, world, site;
    unsigned spin_limit;  // polls of a flag before a wait gives up (kSyncSpinLimit unless the host lowered it)
    // Stamped exchange (flag in data), used when stamp_slots != nullptr: every result word travels
    // as ONE 64-bit word {epoch : value bits} stored into slot stamp_index0 + i of the vector at
    // stamp_slots in every rank's arena (this rank's included); there is no fence, ticket or flag,
    // and the producer does not wait.  epoch = *epoch_dev * epoch_mul + epoch_add.
    unsigned long long* stamp_slots;
    const int* epoch_dev;
    int epoch_mul, epoch_add;
    long long stamp_index0;
};
// The consumer's view of a stamped vector: slot i holds {epoch : bits}; a reader polls (bounded)
// until the epoch it expects is there.  slots == nullptr: the input is an ordinary array.
struct StampIn {
    const unsigned long long* slots;
    const int* epoch_dev;
    int epoch_mul, epoch_add;
    unsigned* err;  // the exchange's error word (ctl + 2 * kSyncMaxSites)
    int site;
    unsigned spin_limit;
};
constexpr unsigned long long kSyncFlagBytes = 4096;  // head of every arena: the flags

// Host-side guard for the launchers: [p, p + bytes) lies inside this rank's arena, behind the flags.
// Peer stores go to the same offset of the peers' arenas, so an output outside the arena would be
// written at an arbitrary place of another GPU's mapping.
inline bool in_arena(const PeerSync& ps, const void* p, unsigned long long bytes) {
    const unsigned char* b = ps.base[ps.rank];
    const unsigned char* q = static_cast<const unsigned char*>(p);
    if (b == nullptr || q < b + kSyncFlagBytes) return false;
    const unsigned long long off = (unsigned long long)(q - b);
    return off <= ps.arena_bytes && bytes <= ps.arena_bytes - off;
}

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned* flag_of(unsigned char* arena, int site, int source) {
    return reinterpret_cast<unsigned*>(arena + (size_t)(site * kSyncMaxRanks + source) * 64);
}
// The address in rank p's arena that corresponds to `local` (a pointer into this rank's arena).
template <class T>
__device__ __forceinline__ T* peer_ptr(const PeerSync& ps, int p, T* local) {
    return reinterpret_cast<T*>(ps.base[p] + (reinterpret_cast<unsigned char*>(local) - ps.base[ps.rank]));
}
// Stores v at `local` and at the same place of every peer's arena.
template <class T>
__device__ __forceinline__ void store_all(const PeerSync& ps, T* local, T v) {
    *local = v;
    for (int p = 0; p < ps.world; ++p)
        if (p != ps.rank) *peer_ptr(ps, p, local) = v;
}
// ---- stamped exchange ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned exchange_epoch(const int* epoch_dev, int mul, int add) {
    return (unsigned)(*reinterpret_cast<const volatile int*>(epoch_dev)) * (unsigned)mul + (unsigned)add;
}
__device__ __forceinline__ void st_stamped(unsigned long long* p, unsigned bits, unsigned epoch) {
    const unsigned long long v = ((unsigned long long)epoch << 32) | bits;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Word `bits` of element `index` of this rank's slice goes to every rank (this one included).
__device__ __forceinline__ void store_stamped_all(const PeerSync& ps, long long index, unsigned bits, unsigned epoch) {
    unsigned long long* local = ps.stamp_slots + ps.stamp_index0 + index;
    for (int p = 0; p < ps.world; ++p) st_stamped(p == ps.rank ? local : peer_ptr(ps, p, local), bits, epoch);
}
__device__ __forceinline__ unsigned long long ld_stamped_raw(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Polls slot p until it carries `epoch` (bounded: a slot that never arrives sets the error word to
// 1 + site, after which every later poll of the exchange gives up at once); returns the value bits.
__device__ __forceinline__ unsigned ld_stamped(const StampIn& in, long long index, unsigned epoch) {
    const unsigned long long* p = in.slots + index;
    unsigned spins = 0;
    for (;;) {
        const unsigned long long v = ld_stamped_raw(p);
        if ((unsigned)(v >> 32) == epoch) return (unsigned)v;
        if ((++spins & 1023u) == 0) {
            if (*reinterpret_cast<volatile unsigned*>(in.err) != 0u) return 0u;
            if (spins > in.spin_limit) {
                atomicCAS(in.err, 0u, (unsigned)in.site + 1u);
                return 0u;
            }
        }
    }
}

// N slots at once: the loads of a round are all in flight together (a lone poll is a round trip to
// L2 at system scope, ~0.6 us; sixteen of them one after the other were most of a consumer's staging
// time); rounds repeat until every live slot carries `epoch`, bounded as above.  bits[i] = 0 on failure.
template <int N>
__device__ __forceinline__ void ld_stamped_n(const StampIn& in, const long long (&index)[N], unsigned live_mask,
                                             unsigned epoch, unsigned (&bits)[N]) {
    unsigned spins = 0;
    for (;;) {
        unsigned long long v[N];
#pragma unroll
        for (int i = 0; i < N; ++i)
            v[i] = ((live_mask >> i) & 1u) ? ld_stamped_raw(in.slots + index[i]) : ((unsigned long long)epoch << 32);
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            ok = ok && (unsigned)(v[i] >> 32) == epoch;
            bits[i] = (unsigned)v[i];
        }
        if (ok) return;
        // Not all here yet: back off before the next round.  Every thread of every CTA polls, and rounds
        // issued back to back would keep L2 busy with polls while the weight streams need it.
        __nanosleep(128);
        if ((++spins & 255u) == 0) {
            bool give_up = *reinterpret_cast<volatile unsigned*>(in.err) != 0u;
            if (!give_up && spins > in.spin_limit) {
                atomicCAS(in.err, 0u, (unsigned)in.site + 1u);
                give_up = true;
            }
            if (give_up) {
#pragma unroll
                for (int i = 0; i < N; ++i) bits[i] = 0u;
                return;
            }
        }
    }
}

// Called by ALL threads of EVERY CTA of the grid after their last peer store.  The last CTA to
// arrive publishes this rank's epoch on every peer and waits (bounded) for the peers' epochs; the
// grid therefore completes only when the whole gathered buffer is in local memory.
__device__ __forceinline__ void peer_finish(const PeerSync& ps) {
    if (ps.world <= 1 || ps.stamp_slots != nullptr) return;  // stamped results need no handshake
    __syncthreads();  // every thread of the CTA has issued its peer stores
    if (threadIdx.x != 0) return;
    __threadfence_system();  // ... and they are performed (cumulatively) before the ticket below
    unsigned* ticket = ps.ctl + kSyncMaxSites + ps.site;
    const unsigned n_ctas = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(ticket, 1u) != n_ctas - 1) return;
    __threadfence();
    *ticket = 0;
    const unsigned epoch = ps.ctl[ps.site] + 1;
    ps.ctl[ps.site] = epoch;
    // Every CTA fenced its peer stores at system scope before taking its ticket, and this thread
    // has observed all tickets: one more fence, then the flags go out as plain system-scope stores
    // (a release store per peer would repeat the flush once per peer).
    __threadfence_system();
    for (int p = 0; p < ps.world; ++p)
        if (p != ps.rank) st_relaxed_sys(flag_of(ps.base[p], ps.site, ps.rank), epoch);
    // Once a wait has run out the exchange is broken (a peer is gone): later calls publish their
    // epoch and return at once instead of each spending the full limit.
    if (*(volatile unsigned*)(ps.ctl + 2 * kSyncMaxSites) != 0u) return;
    for (int p = 0; p < ps.world; ++p) {
        if (p == ps.rank) continue;
        const unsigned* f = flag_of(ps.base[ps.rank], ps.site, p);
        unsigned spins = 0;
        while ((int)(ld_acquire_sys(f) - epoch) < 0) {
            if (++spins > ps.spin_limit) {  // a peer never arrived: report it, keep the context usable
                atomicCAS(ps.ctl + 2 * kSyncMaxSites, 0u, (unsigned)ps.site + 1u);
                return;
            }
        }
    }
}
#endif

// Host side: the exchange the NEXT launch of a kernel that supports it (the Q4_K matvecs, the
// attention merge, the SwiGLU conversion) completes its output with.  Per host thread; consumed
// (reset to "none") by that launch.
void set_next_peer_sync(const PeerSync& ps);
PeerSync take_next_peer_sync();
// The stamped vector the NEXT launch of a kernel that supports it (the Q4_K matvecs with f32 x or
// limb records) reads its input from; same rules.
void set_next_stamp_in(const StampIn& in);
StampIn take_next_stamp_in();

}  // namespace mgpeer
