// Persistent stepping kernel: a whole chunk of simulation steps in ONE cooperative launch.
//
// One block per SM stays resident and loops over the steps. A thread owns four neurons; when
// the network fits (n_pad/4 <= grid threads, e.g. 230 924 neurons on 148 SMs x 512 threads) their
// state lives in registers for the whole launch and HBM/L2 only sees the ring slots, the spike
// lists, the CSR rows of spiking sources and the recorders. Steps inside an exchange window
// need no grid-wide synchronisation at all (a thread touches only its own neurons and ring
// cells); per window there are two grid barriers: after the window's updates, and after the
// delivery of its spikes. That replaces w + 1 kernel launches per window.
//
// Visibility: ring cells and spike lists are written by other SMs between barriers, so every
// read of them goes through L2 (__ldcg); CSR rows and type tables are read-only and use the
// normal path. Spike lists are double buffered by window parity: the list of window k+1 is
// cleared while window k is being delivered.
//
// grid.sync() is the cooperative-groups barrier; the launch is cooperative, so all blocks are
// co-resident by construction (the launch fails cleanly otherwise) and no hand-written spin exists.
#include <cooperative_groups.h>

#include "glif_math.cuh"
#include "persistent.cuh"
#include "philox.cuh"

namespace cg = cooperative_groups;

namespace bmtk {

constexpr int kPT = 512;         // threads per block, one block per SM
constexpr int kSub = 128;        // threads that stream one CSR row together
constexpr int kSmemTypesP = 128;

// 16-byte asynchronous copy global -> shared that caches in L2 only (the ring is written by other SMs)
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr uint32_t kPend = 4096;   // spikes one block can hold for one window

struct BlockShared {
    uint32_t pend_count;           // spikes of the current window collected by this block
    uint32_t base, lbase;          // where this block's spikes go in the global list / log
    uint32_t pend[kPend];          // step_in_window << kSrcBits | global id
};

// Records the fired neurons of this thread in the block's shared-memory list (one shared-memory
// atomic per warp, no global traffic, nothing to wait for).
__device__ __forceinline__ void emit_block(const PersistArgs& a, BlockShared& sh, uint32_t mask, uint32_t ent0) {
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int n = __popc(mask);
    int incl = n;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(full, incl, d);
        if (lane >= d) incl += t;
    }
    uint32_t base = 0;
    if (lane == 31) base = atomicAdd(&sh.pend_count, (uint32_t)incl);
    base = __shfl_sync(full, base, 31);
    uint32_t pos = base + (uint32_t)(incl - n);
#pragma unroll
    for (int j = 0; j < kNeuronsPerThread; ++j) {
        if (mask >> j & 1u) {
            if (pos < kPend) sh.pend[pos] = ent0 + j;
            else atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
            ++pos;
        }
    }
}

// End of a window: the block appends its collected spikes to the global window list (and the spike
// log) with one atomic each, looks up the CSR row of every spiking source and prefetches the row
// into L2 so that the delivery phase, one grid barrier later, finds it there.
__device__ __forceinline__ unsigned long long flush_block(const PersistArgs& a, BlockShared& sh, uint32_t parity,
                                                          unsigned long long win_base) {
    __syncthreads();   // every warp of the block has finished the window's updates
    const uint32_t n = min(sh.pend_count, kPend);
    if (n == 0) return 0ull;   // uniform over the block
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        sh.base = atomicAdd(a.list_counts + parity, n);
        if (a.log_stamp) sh.lbase = atomicAdd(&a.ctl->log_count, n);
    }
    // while those atomics are in flight: row extents and L2 prefetch, one pending spike per warp
    for (uint32_t k = warp; k < n; k += kPT / 32) {
        uint32_t gid, trial;
        split_source(a.ids, sh.pend[k] & kSrcMask, gid, trial);
        const unsigned long long rb = a.rowptr[gid], re = a.rowptr[gid + 1];
        const char* row = reinterpret_cast<const char*>(a.entries + rb);
        for (unsigned long long off = (unsigned long long)lane * 128ull; off < (re - rb) * 8ull; off += 32ull * 128ull)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(row + off));
    }
    __syncthreads();   // base / lbase are known
    for (uint32_t k = threadIdx.x; k < n; k += kPT) {
        const uint32_t e = sh.pend[k];
        const uint32_t gid = e & kSrcMask;   // id in the log: trial * n_pad1 + cell with several trials
        uint32_t row, trial;
        split_source(a.ids, gid, row, trial);
        const unsigned long long rb = a.rowptr[row], re = a.rowptr[row + 1];   // L1 hits now
        const uint32_t pos = sh.base + k;
        if (pos < a.send_cap) a.lists[parity][pos] = make_uint4(e, (uint32_t)(re - rb), (uint32_t)rb, (uint32_t)(rb >> 32));
        else atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
        if (a.log_stamp) {
            const uint32_t lpos = sh.lbase + k;
            if (lpos < a.log_cap) {
                a.log_stamp[lpos] = (uint32_t)(win_base + (e >> kSrcBits) + 1ull);
                a.log_id[lpos] = gid;
            } else {
                atomicOr(&a.ctl->error_flags, kErrLogFull);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) sh.pend_count = 0u;
    return (unsigned long long)n;
}

template <bool THETA, bool IEXT>
__device__ __forceinline__ void do_group(const PersistArgs& a, BlockShared& sh, const TypeConsts* types,
                                         Neuron4<THETA, IEXT>& nr, const int (&pslot)[4], bool valid, uint32_t i0,
                                         unsigned long long step, uint32_t s_in_win, uint32_t sample_base,
                                         const float4* staged = nullptr) {
    uint32_t mask = 0;
    if (valid) {
        const uint32_t np = a.n_pad;
        const uint32_t slot = (uint32_t)(step % a.ring_slots);
        float* ring = a.ring + (size_t)slot * kPorts * np + i0;
        F4 in[kPorts];
        if (staged) {
            // this step's ring slot was copied to shared memory asynchronously (this thread's 4 x 16 B)
#pragma unroll
            for (int p = 0; p < kPorts; ++p) {
                const float4 t = staged[p * kPT];
                in[p] = F4{{t.x, t.y, t.z, t.w}};
            }
        } else {
#pragma unroll
            for (int p = 0; p < kPorts; ++p) in[p] = ld4cg(ring + (size_t)p * np);
        }
        mask = nr.step(types, in);
        const uint32_t li0 = i0 % a.n_pad1;   // cells beyond n_local inside a trial are padding
        if (li0 + kNeuronsPerThread > a.n_local) mask &= (1u << (a.n_local > li0 ? a.n_local - li0 : 0)) - 1u;
        const F4 zero = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int p = 0; p < kPorts; ++p) st4(ring + (size_t)p * np, zero);
        if (a.probe_slot && (step + 1) % a.probe_interval == 0) {
            const unsigned long long sample = (step + 1) / a.probe_interval - 1ull - sample_base;
            if (sample < a.trace_cap) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (pslot[j] >= 0)
                        for (uint32_t v = 0; v < a.n_probe_vars; ++v)
                            a.trace[((size_t)sample * a.n_probe_vars + v) * a.n_probe + pslot[j]] =
                                nr.probe_value(types[nr.ty[j]], j, (a.probe_vars >> (4u * v)) & 15u);
            }
        }
    }
    if (__any_sync(0xffffffffu, mask != 0)) emit_block(a, sh, mask, (s_in_win << kSrcBits) | (a.lo + i0));
}

// ---- several ranks: the exchange is part of this kernel, over peer memory (NVLink / NVSwitch)

__device__ __forceinline__ u64* x_counts(u64* x, uint32_t parity) { return x + parity * kXRanks; }
__device__ __forceinline__ u64* x_inbox(const PersistArgs& a, u64* x, uint32_t parity, uint32_t src_rank) {
    return x + 2 * kXRanks + ((size_t)parity * a.n_ranks + src_rank) * a.xchg_cap;
}

// End of a window with several ranks: the block reserves a range behind this rank's window counter
// and stores its spikes, tagged with the window's sequence number, into inbox[parity][rank] of every
// rank (its own included) with plain 8-byte peer stores; then the spike log, locally.
__device__ __forceinline__ unsigned long long flush_block_multi(const PersistArgs& a, BlockShared& sh, uint32_t parity,
                                                                uint32_t seq, unsigned long long win_base) {
    __syncthreads();
    const uint32_t n = min(sh.pend_count, kPend);
    if (n == 0) return 0ull;
    if (threadIdx.x == 0) {
        sh.base = atomicAdd(a.list_counts + parity, n);
        if (a.log_stamp) sh.lbase = atomicAdd(&a.ctl->log_count, n);
    }
    __syncthreads();
    for (uint32_t k = threadIdx.x; k < n; k += kPT) {
        const uint32_t e = sh.pend[k];
        const uint32_t pos = sh.base + k;
        if (pos < a.xchg_cap) {
            for (uint32_t r = 0; r < a.n_ranks; ++r) st_word(x_inbox(a, a.peers[r], parity, a.rank) + pos, seq, e);
        } else {
            atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
        }
        if (a.log_stamp) {
            const uint32_t lpos = sh.lbase + k;
            if (lpos < a.log_cap) {
                a.log_stamp[lpos] = (uint32_t)(win_base + (e >> kSrcBits) + 1ull);
                a.log_id[lpos] = e & kSrcMask;
            } else {
                atomicOr(&a.ctl->error_flags, kErrLogFull);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) sh.pend_count = 0u;
    return (unsigned long long)n;
}

// After the grid barrier that follows the flush: thread 0 stores this rank's tagged count to every
// rank; the first n_ranks threads of block 0 then wait (bounded) until the count word of every rank
// carries this window's tag. On a time-out the sticky error bit is set and all later waits are
// skipped, so the launch still ends; the host turns the bit into BMTK_E_COMM.

__device__ __forceinline__ void publish_and_wait(const PersistArgs& a, uint32_t parity, uint32_t seq) {
    if (blockIdx.x != 0) return;
    if (threadIdx.x == 0) {
        const uint32_t n = min(__ldcg(a.list_counts + parity), a.xchg_cap);
        for (uint32_t r = 0; r < a.n_ranks; ++r) st_word(x_counts(a.peers[r], parity) + a.rank, seq, n);
    }
    if (threadIdx.x < a.n_ranks && !(__ldcg(&a.ctl->error_flags) & kErrExchangeTimeout)) {
        const u64* w = x_counts(a.peers[a.rank], parity) + threadIdx.x;
        unsigned int spins = 0;
        while ((uint32_t)(ld_word(w) >> 32) != seq) {
            if (++spins > kWaitSpins) {
                atomicOr(&a.ctl->error_flags, kErrExchangeTimeout);
                break;
            }
            __nanosleep(100);
        }
    }
}

// Streams one CSR row [b, b+len) with a group of kSub threads into the ring.
__device__ __forceinline__ void stream_row(const PersistArgs& a, unsigned long long b, unsigned long long en, uint32_t slot0,
                                           uint32_t lane, uint32_t cell0) {
    const uint32_t tb = a.target_bits, tmask = (1u << tb) - 1u;
    const size_t plane = (size_t)a.n_pad;
    float* const ring = a.ring + cell0;
    unsigned long long k = b + lane;
    for (; k + 3ull * kSub < en; k += 4ull * kSub) {
        uint2 e[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e[u] = __ldg(&a.entries[k + (unsigned long long)u * kSub]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            uint32_t slot = slot0 + (e[u].x >> (tb + 2));
            if (slot >= a.ring_slots) slot -= a.ring_slots;
            atomicAdd(ring + ((size_t)slot * kPorts + ((e[u].x >> tb) & 3u)) * plane + (e[u].x & tmask),
                      __uint_as_float(e[u].y));
        }
    }
    for (; k < en; k += kSub) {
        const uint2 e = __ldg(&a.entries[k]);
        uint32_t slot = slot0 + (e.x >> (tb + 2));
        if (slot >= a.ring_slots) slot -= a.ring_slots;
        atomicAdd(ring + ((size_t)slot * kPorts + ((e.x >> tb) & 3u)) * plane + (e.x & tmask), __uint_as_float(e.y));
    }
}

// Delivery of one window: items are the window's spike list (entries carry their row extent), the
// replayed virtual spikes of the window's steps and the on-line Poisson list; a group of kSub
// threads streams one row.
__device__ __forceinline__ void deliver_window(const PersistArgs& a, uint32_t parity, const uint32_t* virt,
                                               unsigned long long win_base, uint32_t win_len) {
    const uint32_t n_rec = min(__ldcg(a.list_counts + parity), a.send_cap);
    uint32_t n_in = 0, in_begin = 0;
    if (a.in_ptr) {
        unsigned long long lo = win_base > a.in_ptr_base ? win_base - a.in_ptr_base : 0ull;
        unsigned long long hi = win_base + win_len > a.in_ptr_base ? win_base + win_len - a.in_ptr_base : 0ull;
        const unsigned long long last = a.in_ptr_len - 1;
        if (lo > last) lo = last;
        if (hi > last) hi = last;
        in_begin = a.in_ptr[lo];
        n_in = a.in_ptr[hi] - in_begin;
    }
    const uint32_t n_virt = virt ? min(__ldcg(virt), a.virt_cap) : 0u;
    const uint32_t total = n_rec + n_in + n_virt;
    const uint32_t sub = threadIdx.x / kSub, lane = threadIdx.x % kSub;
    const uint32_t n_sub = gridDim.x * (kPT / kSub);
    unsigned long long events = 0ull;
    for (uint32_t idx = blockIdx.x * (kPT / kSub) + sub; idx < total; idx += n_sub) {
        if (idx < n_rec) {
            const uint4 e = __ldcg(a.lists[parity] + idx);
            const unsigned long long b = ((unsigned long long)e.w << 32) | e.z;
            const unsigned long long step = win_base + (e.x >> kSrcBits);
            uint32_t row, trial;
            split_source(a.ids, e.x & kSrcMask, row, trial);
            if (lane == 0) events += e.y;
            stream_row(a, b, b + e.y, (uint32_t)(step % a.ring_slots), lane, trial * a.n_pad1);
        } else {
            uint32_t src, row, trial;
            unsigned long long step;
            if (idx < n_rec + n_in) {
                src = a.in_src[in_begin + idx - n_rec];
                step = a.in_step[in_begin + idx - n_rec];
            } else {
                const uint32_t e = __ldcg(virt + 1 + idx - n_rec - n_in);
                src = e & kSrcMask;
                step = win_base + (e >> kSrcBits);
            }
            split_source(a.ids, src, row, trial);
            const unsigned long long b = a.rowptr[row], en = a.rowptr[row + 1];
            if (lane == 0) events += en - b;
            stream_row(a, b, en, (uint32_t)(step % a.ring_slots), lane, trial * a.n_pad1);
        }
    }
    if (events) atomicAdd(&a.ctl->n_events, events);
}

// Delivery with several ranks: the window's spikes of every rank arrive in the local inbox; an entry
// is valid once its tag is this window's (its 8-byte store may land after the count word did, so
// the reader waits for the tag, bounded). Rows are looked up in this rank's CSR, which holds a row
// for every source of the network.
__device__ __forceinline__ void deliver_window_multi(const PersistArgs& a, uint32_t parity, uint32_t seq,
                                                     const uint32_t* virt, unsigned long long win_base, uint32_t win_len) {
    u64* x = a.peers[a.rank];
    uint32_t off[kXRanks + 1];
    off[0] = 0;
    for (uint32_t r = 0; r < a.n_ranks; ++r) {
        const u64 w = ld_word(x_counts(x, parity) + r);
        off[r + 1] = off[r] + ((uint32_t)(w >> 32) == seq ? min((uint32_t)w, a.xchg_cap) : 0u);
    }
    const uint32_t n_rec = off[a.n_ranks];
    uint32_t n_in = 0, in_begin = 0;
    if (a.in_ptr) {
        unsigned long long lo = win_base > a.in_ptr_base ? win_base - a.in_ptr_base : 0ull;
        unsigned long long hi = win_base + win_len > a.in_ptr_base ? win_base + win_len - a.in_ptr_base : 0ull;
        const unsigned long long last = a.in_ptr_len - 1;
        if (lo > last) lo = last;
        if (hi > last) hi = last;
        in_begin = a.in_ptr[lo];
        n_in = a.in_ptr[hi] - in_begin;
    }
    const uint32_t n_virt = virt ? min(__ldcg(virt), a.virt_cap) : 0u;
    const uint32_t total = n_rec + n_in + n_virt;
    const uint32_t sub = threadIdx.x / kSub, lane = threadIdx.x % kSub;
    const uint32_t n_sub = gridDim.x * (kPT / kSub);
    unsigned long long events = 0ull;
    for (uint32_t idx = blockIdx.x * (kPT / kSub) + sub; idx < total; idx += n_sub) {
        uint32_t src;
        unsigned long long step;
        if (idx < n_rec) {
            uint32_t r = 0;
            while (idx >= off[r + 1]) ++r;
            const u64* p = x_inbox(a, x, parity, r) + (idx - off[r]);
            u64 w = ld_word(p);
            unsigned int spins = 0;
            while ((uint32_t)(w >> 32) != seq) {
                if (++spins > kWaitSpins) {
                    atomicOr(&a.ctl->error_flags, kErrExchangeTimeout);
                    break;
                }
                __nanosleep(100);
                w = ld_word(p);
            }
            if ((uint32_t)(w >> 32) != seq) continue;   // uniform over the group: every lane read the same word
            src = (uint32_t)w & kSrcMask;
            step = win_base + ((uint32_t)w >> kSrcBits);
        } else if (idx < n_rec + n_in) {
            src = a.in_src[in_begin + idx - n_rec];
            step = a.in_step[in_begin + idx - n_rec];
        } else {
            const uint32_t e = __ldcg(virt + 1 + idx - n_rec - n_in);
            src = e & kSrcMask;
            step = win_base + (e >> kSrcBits);
        }
        const unsigned long long b = a.rowptr[src], en = a.rowptr[src + 1];
        if (lane == 0) events += en - b;
        stream_row(a, b, en, (uint32_t)(step % a.ring_slots), lane, 0u);   // several ranks: one trial
    }
    if (events) atomicAdd(&a.ctl->n_events, events);
}

template <bool THETA, bool IEXT, bool RESIDENT>
__global__ void __launch_bounds__(kPT, 1) persistent_kernel(const PersistArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ BlockShared sh;
    cg::grid_group grid = cg::this_grid();
    TypeConsts* s_types = reinterpret_cast<TypeConsts*>(smem_raw);
    if (threadIdx.x == 0) sh.pend_count = 0u;
    unsigned long long my_spikes = 0ull;   // block total, kept by thread 0
    __syncthreads();
    const bool use_smem = a.n_types <= kSmemTypesP;
    if (use_smem) {
        const int words = a.n_types * (int)(sizeof(TypeConsts) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.types);
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_types);
        for (int i = threadIdx.x; i < words; i += kPT) dst[i] = src[i];
        __syncthreads();
    }
    const TypeConsts* types = use_smem ? s_types : a.types;
    // RESIDENT: two stage buffers [kPorts][kPT] float4 behind the type table; while step s is computed the
    // ring slot of step s+1 (final inside a window: deliveries happen only at its end) is already on its way
    float4* stage = reinterpret_cast<float4*>(smem_raw + (use_smem ? (sizeof(TypeConsts) * a.n_types + 15) / 16 * 16 : 0));

    const uint32_t nthreads = gridDim.x * kPT;
    const uint32_t gtid = blockIdx.x * kPT + threadIdx.x;
    const uint32_t n_groups = a.n_pad / kNeuronsPerThread;
    const unsigned long long step_base = __ldcg(&a.ctl->step_base);
    const uint32_t sample_base = __ldcg(&a.ctl->sample_base);
    const bool timer = a.profile && gtid == 0;

    // Groups of four neurons are dealt out evenly: block b owns groups [b*gpb, (b+1)*gpb), thread t of
    // the block the t-th of them (and, when gpb > kPT, every kPT-th after it). gpb is a multiple of 32
    // so that a warp is either all neurons or all idle; idle threads take the Poisson cells first.
    const uint32_t gpb = ((n_groups + gridDim.x - 1) / gridDim.x + 31u) & ~31u;
    const uint32_t my_group = blockIdx.x * gpb + threadIdx.x;
    Neuron4<THETA, IEXT> nr;
    int pslot[4] = {-1, -1, -1, -1};
    const bool mine = threadIdx.x < gpb && my_group < n_groups;
    if (RESIDENT && mine) {
        nr.load(a.st, a.n_pad, my_group * kNeuronsPerThread);
        if (a.probe_slot) {
            const int4 q = *reinterpret_cast<const int4*>(a.probe_slot + my_group * kNeuronsPerThread);
            pslot[0] = q.x; pslot[1] = q.y; pslot[2] = q.z; pslot[3] = q.w;
        }
    }
    // Poisson cells are numbered from the last thread of every block downwards
    const uint32_t ptid = (kPT - 1 - threadIdx.x) * gridDim.x + blockIdx.x;

    uint32_t cgi = a.ce_group_begin;       // next clamp group (distinct step with events)
    uint32_t win = 0, s_in_win = 0;
    unsigned long long win_base = step_base;
    unsigned long long t0 = timer ? gtimer() : 0ull;

    for (uint32_t s = 0; s < a.n_steps; ++s) {
        const unsigned long long step = step_base + s;
        uint32_t* virt = a.poisson_thr ? a.virts[win & 1] : nullptr;

        if (IEXT) {
            // Clamp changes effective from this step on; the branch is uniform over the grid. Warps may
            // run a step ahead of their neighbours inside a window, so the change is fenced on both
            // sides: nobody may still be reading i_ext for the previous step when it is applied.
            bool changed = false;
            if (cgi < a.ce_group_end && a.ce_group_step[cgi] <= step) grid.sync();
            while (cgi < a.ce_group_end && a.ce_group_step[cgi] <= step) {
                const uint32_t b = a.ce_group_ptr[cgi], e = a.ce_group_ptr[cgi + 1];
                for (uint32_t k = b + gtid; k < e; k += nthreads)
                    atomicAdd(&a.st.i_ext[a.ce_target[k] - a.lo], a.ce_delta[k]);
                ++cgi;
                changed = true;
            }
            if (changed) {
                grid.sync();
                if (RESIDENT && mine) nr.iex = ld4cg(a.st.i_ext + my_group * kNeuronsPerThread);
            }
        }

        if (RESIDENT) {
            const uint32_t i0 = my_group * kNeuronsPerThread;
            float4* cur = stage + (size_t)(s & 1u) * kPorts * kPT + threadIdx.x;
            if (mine && a.ring_prefetch) {
                if (s_in_win == 0) {
                    const float* r0 = a.ring + (size_t)(step % a.ring_slots) * kPorts * a.n_pad + i0;
#pragma unroll
                    for (int p = 0; p < kPorts; ++p) cp_async16(cur + p * kPT, r0 + (size_t)p * a.n_pad);
                    cp_async_commit();
                }
                cp_async_wait_all();
                if (s_in_win + 1 < a.window && s + 1 < a.n_steps) {
                    float4* nxt = stage + (size_t)((s + 1) & 1u) * kPorts * kPT + threadIdx.x;
                    const float* r1 = a.ring + (size_t)((step + 1) % a.ring_slots) * kPorts * a.n_pad + i0;
#pragma unroll
                    for (int p = 0; p < kPorts; ++p) cp_async16(nxt + p * kPT, r1 + (size_t)p * a.n_pad);
                    cp_async_commit();
                }
            }
            do_group<THETA, IEXT>(a, sh, types, nr, pslot, mine, i0, step, s_in_win, sample_base, a.ring_prefetch ? cur : nullptr);
        } else {
            for (uint32_t t0 = 0; t0 < gpb; t0 += kPT) {
                const uint32_t g = blockIdx.x * gpb + t0 + threadIdx.x;
                const bool valid = t0 + threadIdx.x < gpb && g < n_groups;
                const uint32_t i0 = g * kNeuronsPerThread;
                if (valid) {
                    nr.load(a.st, a.n_pad, i0);
                    if (IEXT) nr.iex = ld4cg(a.st.i_ext + i0);
                    if (a.probe_slot) {
                        const int4 q = *reinterpret_cast<const int4*>(a.probe_slot + i0);
                        pslot[0] = q.x; pslot[1] = q.y; pslot[2] = q.z; pslot[3] = q.w;
                    }
                }
                do_group<THETA, IEXT>(a, sh, types, nr, pslot, valid, i0, step, s_in_win, sample_base);
                if (valid) nr.store(a.st, a.n_pad, i0);
            }
        }

        if (virt) {
            const uint32_t n_virt_all = a.n_virtual * a.n_trials;
            for (uint32_t base = 0; base < n_virt_all; base += nthreads) {
                const uint32_t v = base + ptid;
                int k = 0;
                if (v < n_virt_all) {
                    const uint32_t trial = v / a.n_virtual, cell = v - trial * a.n_virtual;
                    const uint4 thr = a.poisson_thr[cell];
                    const uint32_t x = philox4x32_10(cell, (uint32_t)step, (uint32_t)(step >> 32), a.trial_base + trial,
                                                     (uint32_t)a.seed,
                                                     (uint32_t)(a.seed >> 32)).x;
                    k = (x >= thr.x) + (x >= thr.y) + (x >= thr.z) + (x >= thr.w);
                }
                if (__any_sync(0xffffffffu, k > 0)) {
                    uint32_t tot;
                    const uint32_t pos = warp_reserve(virt, k, &tot);
                    const uint32_t e = (s_in_win << kSrcBits) | (a.ids.n_cells_all + v);
                    for (int j = 0; j < k; ++j) {
                        if (pos + j < a.virt_cap) virt[1 + pos + j] = e;
                        else atomicOr(&a.ctl->error_flags, kErrVirtListFull);
                    }
                    if ((threadIdx.x & 31) == 31) atomicAdd(&a.ctl->n_input_spikes, (unsigned long long)tot);
                }
            }
        }

        ++s_in_win;
        if (s_in_win == a.window || s + 1 == a.n_steps) {
            const bool multi = a.n_ranks > 1;
            const uint32_t seq = a.seq0 + win + 1u;
            const uint32_t par = multi ? (seq & 1u) : (win & 1u);
            my_spikes += multi ? flush_block_multi(a, sh, par, seq, win_base) : flush_block(a, sh, par, win_base);
            const unsigned long long t0b = timer ? gtimer() : 0ull;
            grid.sync();
            if (multi) {
                publish_and_wait(a, par, seq);
                grid.sync();
            }
            const unsigned long long t1 = timer ? gtimer() : 0ull;
            // the other parity's lists were last read one window ago: clear them for the next window
            if (gtid == 0) {
                a.list_counts[par ^ 1u] = 0u;
                if (a.poisson_thr) a.virts[(win + 1) & 1][0] = 0u;
            }
            if (multi) deliver_window_multi(a, par, seq, virt, win_base, s_in_win);
            else deliver_window(a, par, virt, win_base, s_in_win);
            const unsigned long long t1b = timer ? gtimer() : 0ull;
            grid.sync();
            if (timer) {
                const unsigned long long t2 = gtimer();
                a.ctl->t_update_ns += t1 - t0;
                a.ctl->t_prop_ns += t2 - t1;
                a.ctl->t_sync1_ns += t1 - t0b;
                a.ctl->t_sync2_ns += t2 - t1b;
                a.ctl->n_windows += 1ull;
                t0 = t2;
            }
            ++win;
            win_base += s_in_win;
            s_in_win = 0;
        }
    }

    if (RESIDENT && mine) nr.store(a.st, a.n_pad, my_group * kNeuronsPerThread);
    if (gtid == 0) a.ctl->step_base = step_base + a.n_steps;
    if (threadIdx.x == 0 && my_spikes) atomicAdd(&a.ctl->n_spikes, my_spikes);
}

int persistent_max_blocks(int device, bool has_theta, bool has_iext, bool resident, size_t smem) {
    int per_sm = 0, sms = 0;
    const void* f = persistent_kernel_ptr(has_theta, has_iext, resident);
    if (cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, f, kPT, smem) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return per_sm > 0 ? sms : 0;   // one block per SM
}

const void* persistent_kernel_ptr(bool has_theta, bool has_iext, bool resident) {
#define PK(T, I, R) (const void*)persistent_kernel<T, I, R>
    if (has_theta) {
        if (has_iext) return resident ? PK(true, true, true) : PK(true, true, false);
        return resident ? PK(true, false, true) : PK(true, false, false);
    }
    if (has_iext) return resident ? PK(false, true, true) : PK(false, true, false);
    return resident ? PK(false, false, true) : PK(false, false, false);
#undef PK
}

uint32_t persistent_threads_per_block() { return kPT; }

cudaError_t launch_persistent(const PersistArgs& a, bool has_theta, bool has_iext, bool resident, int blocks,
                              cudaStream_t s) {
    const size_t smem = persistent_smem(a.n_types);
    const void* f = persistent_kernel_ptr(has_theta, has_iext, resident);
    cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    PersistArgs copy = a;
    void* args[] = {&copy};
    return cudaLaunchCooperativeKernel(f, dim3(blocks), dim3(kPT), args, smem, s);
}

size_t persistent_smem(int n_types) {
    const size_t t = n_types <= kSmemTypesP ? (sizeof(TypeConsts) * (size_t)n_types + 15) / 16 * 16 : 0;
    return t + 2 * kPorts * kPT * sizeof(float4);   // type table + two ring stage buffers
}

}  // namespace bmtk
