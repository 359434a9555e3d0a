// Pipelined persistent kernel: neuron update and spike delivery run CONCURRENTLY on every SM.
//
// One block of 20 warps per SM (12 where that is enough: more registers a thread, no spills, packed arithmetic in the
// update) stays resident for a whole chunk of steps (cooperative launch, so that all blocks are co-resident). The first warps ("update warps", as many as the network needs at 128
// neurons per warp) own four neurons per thread, state in registers for the whole launch; one or more
// "input warps" draw the Poisson cells / pick up the replayed virtual spikes and queue the block's own
// spikes; with several ranks one "sender warp" stores the block's spikes into the other ranks' exchange
// buffers; the remaining "chunk warps" stream CSR rows into the ring. Time is cut into phases of
// h = floor(min_delay / 2) steps. In phase p
//   * the update warps run the phase's h steps back to back (ring slot in, state update, slot
//     cleared where it received input); a firing lane only appends the spike to a shared-memory list;
//   * the input warps add the chunks of the phase's input spikes to the block's segment of the phase's
//     chunk list (descriptors {first entry, length, ring slot of emission | trial, phase tag}, at most 384 CSR
//     entries each, at positions from a SHARED-memory counter), write the spike log of phase p-1 and,
//     once the update warps have arrived at their named barrier, cut the rows of the block's spiking
//     neurons into chunks as well;
//   * the chunk warps deliver the list of phase p-1, sharing it with their neighbours: chunk j < D of
//     block b is delivered by chunk warp j of block b, chunk D r + i by warp D-1-i of block b + r (D chunk
//     warps per block), so a busy block's spikes spill over to the following SMs. The first D descriptors
//     of a block stay in its shared memory; the neighbours' carry the tag of their phase, so a warp simply
//     loads the few slots it is responsible for (one round trip, no counts to read first) and keeps those
//     with the right tag. A warp copies the entries of all its chunks to shared memory with asynchronous
//     copies (all in flight together) and applies them from there.
// Whatever is emitted in phase p is due min_delay >= 2h steps later, i.e. not before phase p+2 begins,
// so delivering it during phase p+1 neither touches a ring slot that phase reads nor arrives late.
// Compared with update -> barrier -> deliver -> barrier per window, the two latency chains (ring slot
// -> update, and list -> row -> ring reduction) overlap instead of adding up, and no grid barrier is
// left: the update + input warps of phase p+1 wait for the chunk warps of phase p of all blocks, the
// chunk warps of phase p+1 for the update + input warps of phase p of all blocks (side_handover).
// Lists rotate over three buffers: written in phase p, read in p+1, cleared in p+2.
// With several trials over one CSR a launch steps the cells of a few whole trials (PersistArgs::cell0, n_cells); the
// launches of a chunk of steps follow one another over the trials.
//
// Replaces NEST's update/deliver cycle inside nest.Simulate (bmtk/simulator/pointnet/pointsimulator.py:166).
#include <cooperative_groups.h>

#include "glif_math.cuh"
#include "persistent.cuh"
#include "philox.cuh"
#include "pipeline.cuh"

namespace cg = cooperative_groups;

namespace bmtk {

// A block has 20 warps (640 threads, 96 registers each) or 12 (384 threads, up to 168 registers). The first
// PersistArgs::upd_warps of them are update warps - as many as the network needs at 128 neurons per warp, at most
// 16 - and the rest deliver: 13 + 7 of 20 for 230 924 neurons on 148 SMs, 3 + 9 of 12 for 50 000.
constexpr int kBT = 640;            // threads of a block: 20 warps (96 registers a thread), or ...
constexpr int kBTSmall = 384;       // ... 12 warps (up to 168 registers: the update runs without spills) where they are enough
constexpr int kWarps = kBT / 32;
constexpr int kMaxUpdWarps = 16;
constexpr uint32_t kChunk = 384;    // entries of one chunk: the unit of work of one delivery warp (12 per lane). Measured on one
                                    // box: 256 / 320 / 384 / 512 entries = 17.73 / 17.75 / 17.42 / 26.9 ms per simulated second of the
                                    // V1-scale network (most of its rows are 250-350 entries: one chunk instead of two)
constexpr uint32_t kPendP = 2048;   // spikes one block can emit in one phase (its neurons, once each)
constexpr uint32_t kSpill = 4;      // a block's chunks kDW*r .. kDW*r + kDW-1 go to block b + r, for r < kSpill; the rest stay home
constexpr int kSmemTypesPipe = 128;
constexpr int kSmemTypes2 = 64;   // up to this many types the doubled constants for the packed arithmetic are kept as well

// bytes of the type tables in shared memory
__host__ __device__ constexpr size_t type_table_bytes(int n_types) {
    return (n_types <= kSmemTypesPipe ? (sizeof(TypeConsts) * (size_t)n_types + 15) / 16 * 16 : 0) +
           (n_types <= kSmemTypes2 ? sizeof(TypeConsts2) * (size_t)n_types : 0);
}
struct __align__(16) PipeShared {
    uint32_t count[2];              // spikes of the phase with that parity (for the spike log)
    uint32_t chunks[3];             // chunk descriptors this block has added to list L
    uint32_t early[2];              // by phase parity: the producing side's leader saw the other side finished before the hand-over
    uint32_t pad;
    uint4 own[3][kWarps];      // copies of the first descriptors of list L: the ones this block delivers itself
    uint4 sdesc[kWarps][4];    // descriptors of the chunks a warp has staged (see Stager)
    uint2 rows[kMaxUpdWarps * 32 * kNeuronsPerThread];   // {row begin, row length} of this block's neurons
    uint32_t pend[2][kPendP];       // step in phase << kSrcBits | id
};
static_assert(sizeof(PipeShared) % 16 == 0, "the type table behind it is read with 128-bit loads");

// Warps of a block that stream chunks: all but the update and input warps and, with several ranks, the sender warp.
__device__ __forceinline__ uint32_t chunk_warps(const PersistArgs& a) {
    return a.block_warps - a.upd_warps - a.input_warps - (a.n_ranks > 1u ? 1u : 0u);
}

__device__ __forceinline__ uint32_t wrap_slot(uint32_t slot, uint32_t n) { return slot >= n ? slot - n : slot; }

// Third word of a chunk descriptor: ring slot of the emitting step | trial of the source << kTrialShift.
constexpr uint32_t kTrialShift = 20, kSlotMask = (1u << kTrialShift) - 1u;

// Adds the CSR row [begin, begin + len), emitted at ring slot (and in trial) slot0, to this block's segment of list L.
__device__ __forceinline__ void push_chunks(const PersistArgs& a, PipeShared& sh, uint32_t L, uint32_t tag, uint32_t begin,
                                            uint32_t len, uint32_t slot0) {
    const uint32_t n = (len + kChunk - 1) / kChunk;
    if (n == 0) return;
    const uint32_t pos = atomicAdd(&sh.chunks[L], n);
    const uint32_t kDW = chunk_warps(a);
    uint4* seg = a.pipe_seg + ((size_t)L * gridDim.x + blockIdx.x) * a.pipe_seg_cap;
    for (uint32_t c = 0; c < n; ++c) {
        const uint4 d = make_uint4(begin + c * kChunk, min(kChunk, len - c * kChunk), slot0, tag);
        if (pos + c < kDW) sh.own[L][pos + c] = d;   // stays on the SM: no round trip to find it
        else if (pos + c < a.pipe_seg_cap) seg[pos + c] = d;
        else atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
    }
}

// ---- hand-over between the two sides of a phase
// The producing side (update + input warps) of phase p needs the consuming side (chunk warps) of phase
// p-1 finished on EVERY block - its reductions fill the ring slots phase p reads - and the chunk warps
// of phase p need the producing side of phase p-1 finished on every block - its chunk lists. Neither
// needs the other blocks of its OWN side, so instead of one grid barrier per phase each side counts
// its finished blocks in global counters (block-local named barrier, fence, one atomic per block) and
// the leader of the other side polls them. Because a block's side may be a phase or two ahead of
// another block's, arrivals are counted per phase: phase p uses counter p mod 4 and is complete at
// (p / 4 + 1) x blocks (nobody can be four phases ahead). Waits are bounded; a time-out (which a
// cooperative launch rules out short of a bug) sets a sticky error bit and the launch ends.
constexpr unsigned int kSyncSpins = 32000000u;   // far longer than the bounded waits on a peer, which it must outlast

// End of a phase for one side of a block (`n_threads` threads that use named barrier `barrier_id`):
// everybody arrives; the side's leader publishes the block in `mine` and then waits until `other` has
// reached `target` (all blocks' other side have finished the phase); everybody leaves. The fence after
// the barrier is cumulative: it covers the stores and reductions of all threads that arrived.
template <bool MULTI>
__device__ __forceinline__ void side_handover(const PersistArgs& a, uint32_t* mine, const uint32_t* other, uint32_t target,
                                              int barrier_id, uint32_t n_threads, bool leader_warp, bool wait, bool& dead) {
    // barrier.sync, not bar.sync (= barrier.sync.aligned): the leader's warp reaches the second barrier long after the
    // other warps. `leader_warp`: this thread's warp is the side's leader. ALL its lanes poll (one broadcast load): a
    // wait in which lane 0 polled and the others stood by left the warp split in two for the whole next phase.
    asm volatile("barrier.sync %0, %1;" ::"r"(barrier_id), "r"(n_threads) : "memory");
    if (leader_warp) {
        // release: cumulative over what the threads that arrived at the barrier have written (a full
        // fence here would also hold up the other role's warps, which are in the middle of their loads)
        if ((threadIdx.x & 31u) == 0u) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(mine) : "memory");
        if (wait && !dead) {
            // plain polling loads (an acquire load per poll would invalidate the SM's L1 under the other
            // role's feet every time), one acquire load once the count is there
            unsigned int spins = 0;
            while ((int32_t)(*reinterpret_cast<const volatile uint32_t*>(other) - target) < 0) {
                if (++spins > kSyncSpins) {
                    dead = true;
                    break;
                }
            }
            if (dead && (threadIdx.x & 31u) == 0u) atomicOr(&a.ctl->error_flags, kErrSyncTimeout);
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(other) : "memory");
        }
    }
    asm volatile("barrier.sync %0, %1;" ::"r"(barrier_id), "r"(n_threads) : "memory");
}

// Hand-over of the producing side. In networks whose phases are long against their delivery (several steps per phase,
// few events) the chunk warps of every block are done well before the update warps, and the hand-over's own mechanics -
// release, poll, acquire, second barrier: three dependent L2 round trips, 1.3-1.5 us - were a fifth of the phase. So the
// side's leader (lane 0 of the first input warp, which idles while the update warps compute) looks at the other side's
// counter BEFORE the phase ends and leaves what it saw in sh.early; when the other side was done then, the block's
// threads leave after ONE barrier and only the leader stays to publish the block.
template <bool MULTI>
__device__ __forceinline__ void prod_handover(const PersistArgs& a, PipeShared& sh, uint32_t p, uint32_t* mine, const uint32_t* other,
                                              uint32_t target, uint32_t n_threads, bool leader_warp, bool& dead) {
    asm volatile("barrier.sync 2, %0;" ::"r"(n_threads) : "memory");
    const bool done = *reinterpret_cast<volatile uint32_t*>(&sh.early[p & 1u]) != 0u;   // written before the barrier
    if (leader_warp && (threadIdx.x & 31u) == 0u) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(mine) : "memory");
    if (!done) {
        if (leader_warp && !dead) {   // all lanes of the leader's warp: see side_handover
            unsigned int spins = 0;
            while ((int32_t)(*reinterpret_cast<const volatile uint32_t*>(other) - target) < 0) {
                if (++spins > kSyncSpins) {
                    dead = true;
                    break;
                }
            }
            if (dead && (threadIdx.x & 31u) == 0u) atomicOr(&a.ctl->error_flags, kErrSyncTimeout);
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(other) : "memory");
        }
        asm volatile("barrier.sync 2, %0;" ::"r"(n_threads) : "memory");
    }
}

// The leader's early look (a few polls at most: it must not be late for the update warps).
__device__ __forceinline__ void early_look(PipeShared& sh, uint32_t p, const uint32_t* other, uint32_t target, bool wait, bool dead) {
    // (called by all lanes of the leader's warp)
    bool done = !wait;   // the last phase of a launch waits for nobody
    if (wait && !dead) {
        for (int tries = 0; tries < 3 && !done; ++tries)
            done = (int32_t)(*reinterpret_cast<const volatile uint32_t*>(other) - target) >= 0;
        if (done) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(other) : "memory");
        }
    }
    if ((threadIdx.x & 31u) == 0u) *reinterpret_cast<volatile uint32_t*>(&sh.early[p & 1u]) = done ? 1u : 0u;
}

// Option phase_timers: every warp adds the time from the start of its phase to the moment it reaches the hand-over
// to a histogram of its role (0 update, 1 input, 2 chunk warps): 32 bins of 250 ns behind the per-block sums.
__device__ __forceinline__ void hist_add(const PersistArgs& a, uint32_t role, unsigned long long ns) {
    if (!a.blk_prof) return;
    const unsigned long long b = ns / 250ull;
    atomicAdd(a.blk_prof + 4ull * gridDim.x + 32ull * role + (b < 31ull ? b : 31ull), 1ull);
}

struct DeliveryTotals {
    unsigned long long events, inputs, spikes;
    unsigned long long remote_wait_ns, remote_rows_ns;   // option phase_timers, several ranks: this warp's time waiting for the
                                                         // other ranks' count words / fetching and streaming their spikes' rows
};

// Input spikes of the phase [start, start + len) whose first step uses ring slot `slot`: Poisson
// cells (dealt round-robin over the blocks) and this block's share of the replayed spikes, on
// `n_thr` threads of which this is thread `t`.
struct CachedCell {
    uint4 thr;           // Poisson thresholds of the thread's first cell
    uint32_t begin, len; // its CSR row
};

__device__ __forceinline__ void prepare_inputs(const PersistArgs& a, PipeShared& sh, uint32_t L, uint32_t tag,
                                               const CachedCell& cc, unsigned long long start,
                                               uint32_t slot, uint32_t len, uint32_t t, uint32_t n_thr, DeliveryTotals& tot) {
    if (a.poisson_thr) {
        // cell v % n_virtual of trial trial0 + v / n_virtual, over the trials of this launch
        const uint32_t v0 = t * gridDim.x + blockIdx.x, n_virt_all = a.n_virtual * (a.n_cells / a.n_pad1);
        for (uint32_t v = v0; v < n_virt_all; v += n_thr * gridDim.x) {
            const uint32_t tl = v / a.n_virtual, cell = v - tl * a.n_virtual, trial = a.trial0 + tl;
            // the first cell of a thread is kept in registers: no load between the barrier and its spikes
            const uint4 thr = v == v0 ? cc.thr : __ldg(a.poisson_thr + cell);
            for (uint32_t j = 0; j < len; ++j) {
                const unsigned long long step = start + j;
                const uint32_t x = philox4x32_10(cell, (uint32_t)step, (uint32_t)(step >> 32), a.trial_base + trial, (uint32_t)a.seed,
                                                 (uint32_t)(a.seed >> 32)).x;
                const uint32_t k = (x >= thr.x) + (x >= thr.y) + (x >= thr.z) + (x >= thr.w);
                if (k) {
                    uint32_t rb = cc.begin, rl = cc.len;
                    if (v != v0) {
                        const unsigned long long b0 = a.rowptr[a.n_global + cell], b1 = a.rowptr[a.n_global + cell + 1];
                        rb = (uint32_t)b0;
                        rl = (uint32_t)(b1 - b0);
                    }
                    for (uint32_t c = 0; c < k; ++c)
                        push_chunks(a, sh, L, tag, rb, rl, wrap_slot(slot + j, a.ring_slots) | (trial << kTrialShift));
                    tot.inputs += k;
                }
            }
        }
    }
    if (a.in_ptr) {
        unsigned long long lo = start > a.in_ptr_base ? start - a.in_ptr_base : 0ull;
        unsigned long long hi = start + len > a.in_ptr_base ? start + len - a.in_ptr_base : 0ull;
        const unsigned long long last = a.in_ptr_len - 1;
        if (lo > last) lo = last;
        if (hi > last) hi = last;
        const uint32_t in_begin = a.in_ptr[lo], in_end = a.in_ptr[hi];
        for (uint32_t idx = in_begin + t * gridDim.x + blockIdx.x; idx < in_end; idx += n_thr * gridDim.x) {
            const uint32_t src = a.in_src[idx];
            const unsigned long long rb = a.rowptr[src], re = a.rowptr[src + 1];
            push_chunks(a, sh, L, tag, (uint32_t)rb, (uint32_t)(re - rb),
                        wrap_slot(slot + (uint32_t)(a.in_step[idx] - start), a.ring_slots));
        }
    }
}

// ---- staged streaming: a warp that has several chunks to deliver (its own, a neighbour's spill-over, the rows of
// remote spikes) would pay one DRAM round trip per chunk if it streamed them one after the other, and holding two
// chunks' entries in registers spills. Instead the entries of up to kStage chunks are copied to the warp's own piece
// of shared memory with asynchronous copies (no registers, all in flight together) and applied from there as each
// copy group lands.
constexpr int kStage = 3;
struct Stager {
    uint2* buf;       // [kStage][kChunk] of this warp
    uint4* desc;      // [kStage]
    uint32_t m;       // chunks staged and not yet applied
};

__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sa), "l"(gmem) : "memory");
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}

__device__ __forceinline__ void stage_flush(const PersistArgs& a, Stager& s, uint32_t lane) {
    const uint32_t tb = a.target_bits, tmask = (1u << tb) - 1u;
    const size_t plane = (size_t)a.n_pad;
    for (uint32_t i = 0; i < s.m; ++i) {
        switch (s.m - 1u - i) {   // copy groups still allowed in flight: those of the chunks behind this one
            case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
            case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
            default: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        }
        __syncwarp();
        const uint4 d = s.desc[i];
        const uint2* src = s.buf + i * kChunk;
        const uint32_t slot0 = d.z & kSlotMask;
        float* const cells = a.ring + (size_t)(d.z >> kTrialShift) * a.n_pad1;   // the source's trial
        for (uint32_t u = lane; u < d.y; u += 32u) {   // a lane applies the entries it copied itself
            const uint2 e = src[u];
            uint32_t slot = slot0 + (e.x >> (tb + 2));
            if (slot >= a.ring_slots) slot -= a.ring_slots;
            atomicAdd(cells + ((size_t)slot * kPorts + ((e.x >> tb) & 3u)) * plane + (e.x & tmask), __uint_as_float(e.y));
        }
    }
    __syncwarp();
    s.m = 0;
}

__device__ __forceinline__ void stage_add(const PersistArgs& a, Stager& s, const uint4 d, uint32_t lane) {
    if ((unsigned long long)d.x + d.y > a.n_entries || d.y > kChunk || (d.z & kSlotMask) >= a.ring_slots ||
        (d.z >> kTrialShift) >= a.n_trials) {
        if (lane == 0) atomicOr(&a.ctl->error_flags, kErrBadChunk);
        return;
    }
    uint2* dst = s.buf + s.m * kChunk;
    for (uint32_t u = lane; u < d.y; u += 32u) cp_async8(dst + u, a.entries + d.x + u);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (lane == 0) s.desc[s.m] = d;
    if (++s.m == (uint32_t)kStage) stage_flush(a, s, lane);
}

__device__ __forceinline__ void deliver_chunk(const PersistArgs& a, Stager& s, const uint4 d, uint32_t lane) {
    stage_add(a, s, d, lane);
}

// Delivery of list L (written in the phase with tag `tag`) by warp `w` of this block's delivery
// warps: chunk kDW*r + w of block b - r for r < kSpill, found by their tag, then this block's own
// chunks beyond kDW * kSpill. Called by whole warps.
__device__ __forceinline__ void deliver_list(const PersistArgs& a, PipeShared& sh, Stager& sg, uint32_t L, uint32_t tag, uint32_t w,
                                             uint32_t lane, DeliveryTotals& tot) {
    const uint32_t G = gridDim.x, kDW = chunk_warps(a);
    // the neighbours' descriptors are requested first, then this block's own chunk (descriptor in shared
    // memory) is streamed while they are on their way
    uint4 d = make_uint4(0u, 0u, 0u, 0u);
    if (lane >= 1 && lane < kSpill && lane < G) {
        const uint32_t src = (blockIdx.x + G - lane) % G;
        // a neighbour's spill-over is taken from the far end of the warps: its chunk kDW r + i goes to warp kDW-1-i of
        // block b + r, whose own chunks fill its warps from 0 upwards, so the two rarely meet in one warp
        d = __ldcg(a.pipe_seg + ((size_t)L * G + src) * a.pipe_seg_cap + kDW * lane + (kDW - 1u - w));
    }
    unsigned long long events = 0ull;
    if (w < min(sh.chunks[L], a.pipe_seg_cap)) {
        const uint4 c = sh.own[L][w];
        events += c.y;
        deliver_chunk(a, sg, c, lane);
    }
    uint32_t valid = __ballot_sync(0xffffffffu, lane >= 1 && lane < kSpill && lane < G && d.w == tag);
    while (valid) {
        const int r = __ffs(valid) - 1;
        valid &= valid - 1u;
        uint4 c;
        c.x = __shfl_sync(0xffffffffu, d.x, r);
        c.y = __shfl_sync(0xffffffffu, d.y, r);
        c.z = __shfl_sync(0xffffffffu, d.z, r);
        c.w = tag;
        events += c.y;
        deliver_chunk(a, sg, c, lane);
    }
    // a block with more than kDW * kSpill chunks (or fewer blocks than kSpill) keeps the rest
    const uint32_t n_own = min(sh.chunks[L], a.pipe_seg_cap);
    const uint32_t first = kDW * min(kSpill, G);
    for (uint32_t j = first + w; j < n_own; j += kDW) {
        const uint4 c = __ldcg(a.pipe_seg + ((size_t)L * G + blockIdx.x) * a.pipe_seg_cap + j);
        events += c.y;
        deliver_chunk(a, sg, c, lane);
    }
    if (lane == 0) tot.events += events;
}

// Several ranks: what block b of every other rank emitted in the phase with index k mod 4 and tag `tag` is
// delivered by block b here. Lane r of every chunk warp waits (bounded) for the tagged count word of rank r, so
// the waits on the different ranks overlap; the ranks' entries then form ONE list (rank 0's, rank 1's, ...) that
// is dealt round-robin to the block's chunk warps - a rank contributes one or two spikes per block and phase, and
// dealing every rank's entries separately would leave warp 0 with a row of every rank and the others idle. For
// its entry the warp waits for the entry's tag (its store may trail the count word), looks up the row of the
// spiking neuron in THIS rank's CSR (all sources have a row, the targets are local) and streams it.
__device__ __forceinline__ void deliver_remote(const PersistArgs& a, Stager& sg, u64* xp, uint32_t k, uint32_t tag, uint32_t prev_slot,
                                               uint32_t w, uint32_t n_cw, uint32_t lane, DeliveryTotals& tot, bool& dead) {
    unsigned long long events = 0ull;
    uint32_t my_n = 0;
    const unsigned long long t_in = a.profile ? gtimer() : 0ull;
    {
        // every lane stays in the loop until all the lanes with a rank to wait for have their word (a wait that only
        // some lanes of a warp spin in can leave the warp split for what follows)
        const bool need = lane < a.n_ranks && lane != a.rank && !dead;
        const u64* p = xp_cnt(xp, k, need ? lane : a.rank, blockIdx.x);
        bool have = !need;
        u64 cw = 0;
        unsigned int spins = 0;
        for (;;) {
            if (!have) {
                cw = ld_word(p);
                have = (uint32_t)(cw >> 32) == tag;
            }
            if (__all_sync(0xffffffffu, have)) break;
            if (++spins > kWaitSpins) {
                if (!have) atomicOr(&a.ctl->error_flags, kErrExchangeTimeout);
                dead = true;
                break;
            }
            __nanosleep(50);
        }
        if (need && have) my_n = min((uint32_t)cw, kXPipeSeg);
    }
    const unsigned long long t_counts = a.profile ? gtimer() : 0ull;
    // exclusive prefix of the ranks' counts over the lanes
    uint32_t incl = my_n;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, dlt);
        if (lane >= (uint32_t)dlt) incl += t;
    }
    const uint32_t my_off = incl - my_n;
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    // (dealt from the LAST chunk warp downwards: the block's own chunks fill the warps from the first upwards)
    for (uint32_t j = n_cw - 1u - w; j < total; j += n_cw) {
        const uint32_t owner = __ballot_sync(0xffffffffu, my_n != 0u && my_off <= j && j < my_off + my_n);
        const int r = __ffs(owner) - 1;   // exactly one lane holds j
        const uint32_t i = j - __shfl_sync(0xffffffffu, my_off, r);
        const u64* ent = xp_ent(xp, k, (uint32_t)r, blockIdx.x, a.n_ranks, gridDim.x);
        u64 e = 0;
        {
            unsigned int spins = 0;   // all lanes read the entry's word (a broadcast)
            while ((uint32_t)((e = ld_word(ent + i)) >> 32) != tag) {
                if (++spins > kWaitSpins) {
                    if (lane == 0) atomicOr(&a.ctl->error_flags, kErrExchangeTimeout);
                    break;
                }
                __nanosleep(50);
            }
        }
        e = __shfl_sync(0xffffffffu, e, 0);
        if ((uint32_t)(e >> 32) != tag) continue;
        const uint32_t src = (uint32_t)e & kSrcMask;
        const unsigned long long rb = a.rowptr[src], re = a.rowptr[src + 1];
        const uint32_t slot0 = wrap_slot(prev_slot + ((uint32_t)e >> kSrcBits), a.ring_slots);
        events += re - rb;
        for (unsigned long long c = rb; c < re; c += kChunk)
            deliver_chunk(a, sg, make_uint4((uint32_t)c, (uint32_t)min((unsigned long long)kChunk, re - c), slot0, 0u), lane);
    }
    stage_flush(a, sg, lane);
    if (lane == 0) tot.events += events;
    if (a.profile && lane == 0) {
        tot.remote_wait_ns += t_counts - t_in;
        tot.remote_rows_ns += gtimer() - t_counts;
    }
}

// The block's neuron spikes of the phase with parity `par` (collected in sh.pend by the update warps) are turned
// into chunk descriptors by the input threads (`n_thr` of them, this is thread `t`), one spike per thread. The row of a neuron is kept in sh.rows under the index of the update
// thread that owns it: group g of four neurons belongs to chunk g / 32 = warp x gridDim.x + block.
__device__ __forceinline__ void queue_block_spikes(const PersistArgs& a, PipeShared& sh, uint32_t L, uint32_t tag, uint32_t par,
                                                   uint32_t slot, uint32_t t, uint32_t n_thr) {
    const uint32_t n = min(sh.count[par], kPendP);
    for (uint32_t k = t; k < n; k += n_thr) {
        const uint32_t ent = sh.pend[par][k];
        const uint32_t cell = (ent & kSrcMask) - a.lo, local = cell - a.cell0, grp = local >> 2;
        const uint32_t thr = ((grp >> 5) / gridDim.x) * 32u + (grp & 31u);
        const uint2 r = sh.rows[thr * kNeuronsPerThread + (local & 3u)];
        const uint32_t trial = a.n_trials > 1u ? cell / a.n_pad1 : 0u;
        push_chunks(a, sh, L, tag, r.x, r.y, wrap_slot(slot + (ent >> kSrcBits), a.ring_slots) | (trial << kTrialShift));
    }
}

// Spike log of the phase whose list has parity q (stamps count from prev_start); one warp. Every block
// logs into its own segment [blockIdx.x * log_seg_cap, ...) of the log arrays at a position the warp
// carries in a register (`pos`, same on all lanes): no atomic, no round trip. The segments are laid end
// to end when the host drains the log.
__device__ __forceinline__ void write_log(const PersistArgs& a, PipeShared& sh, uint32_t lane, uint32_t n_rec, uint32_t q,
                                          unsigned long long prev_start, uint32_t& pos) {
    const size_t seg = (size_t)blockIdx.x * a.log_seg_cap;
    for (uint32_t k = lane; k < n_rec; k += 32) {
        const uint32_t e = sh.pend[q][k];
        if (pos + k < a.log_seg_cap) {
            a.log_stamp[seg + pos + k] = (uint32_t)(prev_start + (e >> kSrcBits) + 1ull);
            a.log_id[seg + pos + k] = e & kSrcMask;
        } else {
            atomicOr(&a.ctl->error_flags, kErrLogFull);
        }
    }
    pos = min(pos + n_rec, a.log_seg_cap);
}

__device__ __forceinline__ void log_previous_phase(const PersistArgs& a, PipeShared& sh, uint32_t lane, uint32_t q,
                                                   unsigned long long prev_start, uint32_t& log_pos, DeliveryTotals& tot) {
    const uint32_t n_rec = min(sh.count[q], kPendP);
    if (a.log_stamp && n_rec) write_log(a, sh, lane, n_rec, q, prev_start, log_pos);
    __syncwarp();
    if (lane == 0) {
        sh.count[q] = 0u;    // the update warps append to it again in the next phase
        tot.spikes += n_rec;
    }
}

template <bool THETA, bool IEXT, bool MULTI, int BT>
__global__ void __launch_bounds__(BT, 1) pipelined_kernel(const PersistArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    cg::grid_group grid = cg::this_grid();
    PipeShared& sh = *reinterpret_cast<PipeShared*>(smem_raw);
    TypeConsts* s_types = reinterpret_cast<TypeConsts*>(smem_raw + sizeof(PipeShared));
    const bool use_smem = a.n_types <= kSmemTypesPipe;
    if (threadIdx.x == 0) {
        sh.count[0] = sh.count[1] = 0u;
        sh.chunks[0] = sh.chunks[1] = sh.chunks[2] = 0u;
    }
    if (use_smem) {
        const int words = a.n_types * (int)(sizeof(TypeConsts) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.types);
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_types);
        for (int i = threadIdx.x; i < words; i += BT) dst[i] = src[i];
    }
    const TypeConsts* types = use_smem ? s_types : a.types;
    // the constants of the integrating step once more, doubled, for the packed arithmetic
    // (in the 12-warp block only: with the 96 registers of the 20-warp block the packed code spills more and came out
    // 2-5 % slower than the scalar code, against 11 % faster where registers are plentiful; tune 1 / 2 force either)
    const bool packed = a.n_types <= kSmemTypes2 && (a.tune & 2u ? true : a.tune & 1u ? false : BT == kBTSmall);
    TypeConsts2* const s_types2 = reinterpret_cast<TypeConsts2*>(smem_raw + sizeof(PipeShared) +
                                                                 (sizeof(TypeConsts) * (size_t)a.n_types + 15) / 16 * 16);
    if (packed) {
        const float* src = reinterpret_cast<const float*>(a.types);
        float2* dst = reinterpret_cast<float2*>(s_types2);
        for (int i = threadIdx.x; i < a.n_types * kDupFloats; i += BT) {
            const float c = src[(i / kDupFloats) * (int)(sizeof(TypeConsts) / 4) + i % kDupFloats];
            dst[i] = make_float2(c, c);
        }
    }
    // behind the type tables: the warps' staging buffers for CSR entries
    uint2* const s_stage = reinterpret_cast<uint2*>(smem_raw + sizeof(PipeShared) + type_table_bytes(a.n_types));

    const uint32_t kUT = 32u * a.upd_warps, kDT = BT - kUT, kDW = kDT / 32u;
    // behind the chunk warps' staging buffers: two buffers of ring cells per update thread (option ring_stage)
    float4* const s_ring = reinterpret_cast<float4*>(s_stage + (size_t)chunk_warps(a) * kStage * kChunk);
    // delivery warps: kCW stream chunks, then the input warps, then (several ranks) the sender warp
    const uint32_t kCW = kDW - a.input_warps - (MULTI ? 1u : 0u);
    const uint32_t n_prod_threads = kUT + 32u * a.input_warps, n_cons_threads = 32u * kCW;
    // named barrier 3: the update warps arrive when their phase is done; the input warps (which queue the block's
    // spikes) and the sender warp wait on it
    const uint32_t n_bar3 = n_prod_threads + (MULTI ? 32u : 0u);
    constexpr bool multi = MULTI;   // several ranks: a separate instantiation keeps the exchange out of the one-rank kernel
    uint32_t* const cnt_prod = a.pipe_sync;        // [4] blocks of this rank whose update + input warps finished phase p (index p mod 4)
    uint32_t* const cnt_cons = a.pipe_sync + 4;    // [4] blocks of this rank whose chunk warps finished phase p
    u64* const xp_self = multi ? a.peers[a.rank] + a.xp_off : nullptr;
    bool sync_dead = false;
    const bool is_upd = threadIdx.x < kUT;
    const uint32_t dtid = threadIdx.x - kUT;
    const uint32_t n_groups = a.n_cells / kNeuronsPerThread;
    const unsigned long long step_base = __ldcg(&a.ctl->step_base);
    const uint32_t sample_base = __ldcg(&a.ctl->sample_base);
    // Neurons are dealt to the update warps in chunks of 128 (32 lanes x 4), round-robin over the blocks:
    // chunk c belongs to warp c / gridDim.x of block c % gridDim.x. Neurons are sorted by type, so every
    // block gets its share of every type.
    const uint32_t my_group = ((threadIdx.x >> 5) * gridDim.x + blockIdx.x) * 32u + (threadIdx.x & 31u);
    const uint32_t i0 = a.cell0 + my_group * kNeuronsPerThread;   // first of the thread's four cells (trial-major with several trials)
    const uint32_t li0 = a.n_trials > 1u ? i0 % a.n_pad1 : i0;    // ... inside its trial
    const bool mine = is_upd && my_group < n_groups;
    const bool timer_u = a.profile && threadIdx.x == 0;      // every block times itself; block 0's sums also go to the control block
    const bool timer_d = a.profile && threadIdx.x == kUT;

    // clamp changes already in force at the first step of this launch
    uint32_t cgi = a.ce_group_begin;
    if (IEXT) {
        bool any = false;
        while (cgi < a.ce_group_end && a.ce_group_step[cgi] <= step_base) {
            const uint32_t b = a.ce_group_ptr[cgi], e = a.ce_group_ptr[cgi + 1];
            for (uint32_t k = b + blockIdx.x * BT + threadIdx.x; k < e; k += gridDim.x * BT)
                atomicAdd(&a.st.i_ext[a.ce_target[k] - a.lo], a.ce_delta[k]);
            ++cgi;
            any = true;
        }
        if (any) grid.sync();
    }
    __syncthreads();

    const uint32_t S = a.ring_slots;
    uint32_t slot = (uint32_t)(step_base % S);   // ring slot of the phase's first step
    uint32_t s = 0, p = 0;
    // phase timers (option): block 0's first update and first delivery thread sum their busy and waiting
    // time in registers and add them to the control block when the launch ends
    unsigned long long t_mark = (timer_u || timer_d) ? gtimer() : 0ull;
    unsigned long long acc_work = 0ull, acc_wait = 0ull, acc_rows = 0ull;

    // Both roles walk the same phase schedule: h steps, cut short where a clamp change takes effect
    // (a change always starts a phase) and at the end of the launch.
#define PIPE_PHASE_BEGIN()                                                   \
    const unsigned long long start = step_base + s;                          \
    uint32_t len = min(a.half, a.n_steps - s);                               \
    bool clamp_next = false;                                                 \
    if (IEXT && cgi < a.ce_group_end) {                                      \
        const unsigned long long gs = a.ce_group_step[cgi]; /* > start */    \
        /* a change that takes effect on the first step AFTER this launch is  \
           left to the next launch's prologue (applying it here as well      \
           would add it twice)                                                \
        */                                                                   \
        if (gs - start < (unsigned long long)len ||                          \
            (gs - start == (unsigned long long)len && s + len < a.n_steps)) {\
            len = (uint32_t)(gs - start);                                    \
            clamp_next = true;                                               \
        }                                                                    \
    }                                                                        \
    const uint32_t par = p & 1u;                                             \
    const uint32_t L = p % 3u;                                               \
    const uint32_t tag = (uint32_t)start + 1u; /* of what this phase emits */

    if (is_upd) {
        // ================= update warps
        Neuron4<THETA, IEXT> nr;
        bool clamp_now = false;
        if (mine) {
            nr.load(a.st, a.n_pad, i0);
            if (IEXT) nr.iex = ld4cg(a.st.i_ext + i0);
#pragma unroll
            for (int j = 0; j < kNeuronsPerThread; ++j) {
                const uint32_t row = a.lo + min(li0 + (uint32_t)j, a.n_local - 1u);   // (cells beyond n_local are padding and never spike)
                const unsigned long long rb = a.rowptr[row], re = a.rowptr[row + 1];
                sh.rows[threadIdx.x * kNeuronsPerThread + j] = make_uint2((uint32_t)rb, (uint32_t)(re - rb));
            }
        }
        // probes: a sample is taken after the step that ends a recording interval
        uint32_t pctr = 0;                 // (step + 1) mod interval of the next step to run
        unsigned long long sample = 0;     // sample that step writes when pctr == 0, relative to the drained ones
        if (a.probe_slot) {
            pctr = (uint32_t)((step_base + 1ull) % a.probe_interval);
            sample = (step_base + 1ull) / a.probe_interval - 1ull - sample_base;
            if (pctr != 0) sample += 1ull;   // the next multiple of the interval
        }
        // phases of several steps: the ring cells of step j + 1 (final since the phase began) are copied to shared
        // memory while step j computes, so that only the first step of a phase waits for an L2 round trip
        float4* const my_ring = s_ring + threadIdx.x;   // [buffer][port][update thread]
        while (s < a.n_steps) {
            PIPE_PHASE_BEGIN()
            const unsigned long long t_warp = a.profile ? gtimer() : 0ull;
            if (IEXT && clamp_now) {
                if (mine) nr.iex = ld4cg(a.st.i_ext + i0);
                clamp_now = false;
            }
            uint32_t sl = slot;
            for (uint32_t j = 0; j < len; ++j) {
                uint32_t mask = 0;
                if (mine) {
                    float* ring = a.ring + (size_t)sl * kPorts * a.n_pad + i0;
                    const bool ahead = a.ring_stage && j + 1u < len;
                    if (ahead) {
                        const float* nxt = a.ring + (size_t)wrap_slot(sl + 1u, S) * kPorts * a.n_pad + i0;
#pragma unroll
                        for (int pt = 0; pt < kPorts; ++pt)
                            cp_async16(my_ring + (((j + 1u) & 1u) * kPorts + pt) * kUT, nxt + (size_t)pt * a.n_pad);
                        asm volatile("cp.async.commit_group;" ::: "memory");
                    }
                    F4 in[kPorts];
                    if (a.ring_stage && j > 0u) {
                        if (ahead) asm volatile("cp.async.wait_group 1;" ::: "memory");
                        else asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
                        for (int pt = 0; pt < kPorts; ++pt) {
                            const float4 t = my_ring[((j & 1u) * kPorts + pt) * kUT];
                            in[pt] = F4{{t.x, t.y, t.z, t.w}};
                        }
                    } else {
#pragma unroll
                        for (int pt = 0; pt < kPorts; ++pt) in[pt] = ld4cg(ring + (size_t)pt * a.n_pad);
                    }
                    mask = packed ? nr.step_packed(types, s_types2, in) : nr.step(types, in);
                    if (li0 + kNeuronsPerThread > a.n_local) mask &= (1u << (a.n_local > li0 ? a.n_local - li0 : 0)) - 1u;
                    const F4 zero = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int pt = 0; pt < kPorts; ++pt) {
                        const bool nz = in[pt].v[0] != 0.f || in[pt].v[1] != 0.f || in[pt].v[2] != 0.f || in[pt].v[3] != 0.f;
                        if (nz) st4(ring + (size_t)pt * a.n_pad, zero);   // most cells are still zero
                    }
                }
                if (a.profile && j + 1 == len) {
                    const bool any = __any_sync(0xffffffffu, mask != 0u);
                    if ((threadIdx.x & 31u) == 0u) {
                        const unsigned long long dt_ = gtimer() - t_warp;
                        hist_add(a, any ? 4u : 3u, dt_);
                        if (a.blk_prof) a.blk_prof[4ull * gridDim.x + 160ull + 16ull * blockIdx.x + (threadIdx.x >> 5)] += dt_;
                    }
                }
                if (a.probe_slot) {
                    if (pctr == 0) {
                        if (mine && sample < a.trace_cap) {
                            // (the trace columns of the four neurons are fetched when a sample is due, not kept in registers)
                            const int4 qd = __ldg(reinterpret_cast<const int4*>(a.probe_slot + i0));
                            const int pslot[4] = {qd.x, qd.y, qd.z, qd.w};
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                if (pslot[jj] >= 0)
                                    for (uint32_t v = 0; v < a.n_probe_vars; ++v)
                                        a.trace[((size_t)sample * a.n_probe_vars + v) * a.n_probe + pslot[jj]] =
                                            nr.probe_value(types[nr.ty[jj]], jj, (a.probe_vars >> (4u * v)) & 15u);
                        }
                        ++sample;
                    }
                    if (++pctr == a.probe_interval) pctr = 0;
                }
                if (mask) {
                    // spikes are rare: each firing lane appends for itself
#pragma unroll
                    for (int jj = 0; jj < kNeuronsPerThread; ++jj) {
                        if (mask >> jj & 1u) {
                            const uint32_t pos = atomicAdd(&sh.count[par], 1u);
                            const uint32_t ent = (j << kSrcBits) | (a.lo + i0 + jj);
                            if (pos < kPendP) sh.pend[par][pos] = ent;
                            else atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
                            // the input warps queue the spike at the end of the phase (queue_block_spikes): done here, by
                            // the one firing lane with the warp's state in registers around it, it cost the whole warp more
                            // than a microsecond (registers spilled around a path that is rarely taken miss every cache)
                        }
                    }
                }
                sl = wrap_slot(sl + 1u, S);
            }
            // done with phase p; the next one needs the chunk warps of phase p finished everywhere (ring slots final)
            asm volatile("barrier.arrive 3, %0;" ::"r"(n_bar3) : "memory");   // this phase's spikes are in sh.pend
            const unsigned long long t_work = timer_u ? gtimer() : 0ull;
            if (a.profile && (threadIdx.x & 31u) == 0u) {
                const unsigned long long now = gtimer();
                hist_add(a, 0u, now - t_warp);
            }
            prod_handover<MULTI>(a, sh, p, cnt_prod + (p & 3u), cnt_cons + (p & 3u), (p / 4u + 1u) * gridDim.x, n_prod_threads, false,
                                 sync_dead);
            if (timer_u) {
                const unsigned long long t_end = gtimer();
                acc_work += t_end - t_mark;   // the whole phase; acc_wait is the part spent in the hand-over
                acc_wait += t_end - t_work;
                t_mark = t_end;
            }
            if (IEXT && clamp_next) {
                while (cgi < a.ce_group_end && a.ce_group_step[cgi] <= start + len) ++cgi;
                clamp_now = true;   // reload i_ext once the chunk warps that applied the change are done
            }
            slot = (uint32_t)((slot + len) % S);
            s += len;
            ++p;
        }
        if (mine) nr.store(a.st, a.n_pad, i0);
        if (blockIdx.x == 0 && threadIdx.x == 0 && a.advance_clock) a.ctl->step_base = step_base + a.n_steps;
        if (timer_u) {
            if (blockIdx.x == 0) {
                a.ctl->t_update_ns += acc_work;
                a.ctl->t_sync1_ns += acc_wait;
                a.ctl->n_windows += p;
            }
            if (a.blk_prof) {
                a.blk_prof[4 * blockIdx.x + 0] += acc_work - acc_wait;
                a.blk_prof[4 * blockIdx.x + 1] += acc_wait;
            }
        }
    } else {
        // ================= delivery warps
        const uint32_t lane = dtid & 31u, dwarp = dtid >> 5;
        const bool input_role = dwarp >= kCW && dwarp < kCW + a.input_warps;
        const bool sender_role = MULTI && dwarp == kCW + a.input_warps;
        const uint32_t log_warp = kCW;   // the first input warp (a block always has one)
        const uint32_t log_pos0 = (a.log_append && a.log_stamp) ? a.log_seg_cnt[blockIdx.x] : 0u;
        uint32_t log_pos = log_pos0;   // entries in this block's log segment
        const uint32_t it = dtid - 32u * kCW, n_it = 32u * a.input_warps;   // input thread index / count
        unsigned long long prev_start = step_base;
        uint32_t prev_slot = slot;   // ring slot of the previous phase's first step
        DeliveryTotals tot = {0ull, 0ull, 0ull, 0ull, 0ull};
        Stager sg;
        sg.buf = s_stage + (size_t)min(dwarp, kCW - 1u) * kStage * kChunk;   // only chunk warps stage (input / sender warps never use it)
        sg.desc = sh.sdesc[threadIdx.x >> 5];
        sg.m = 0;
        CachedCell cc = {make_uint4(0u, 0u, 0u, 0u), 0u, 0u};
        if (input_role && a.poisson_thr && it * gridDim.x + blockIdx.x < a.n_virtual * (a.n_cells / a.n_pad1)) {
            const uint32_t v0 = (it * gridDim.x + blockIdx.x) % a.n_virtual;
            cc.thr = __ldg(a.poisson_thr + v0);
            const unsigned long long b0 = a.rowptr[a.n_global + v0], b1 = a.rowptr[a.n_global + v0 + 1];
            cc.begin = (uint32_t)b0;
            cc.len = (uint32_t)(b1 - b0);
        }
        if (sender_role) {
            // ---- several ranks: this warp alone talks to the other GPUs. It takes the block's spikes of a phase as soon
            // as the update warps are done with it and stores them, then the tagged count word, into the exchange buffer
            // of every other rank (plain peer stores, fire and forget). It joins neither hand-over: the release with
            // which a side publishes its phase waits for the writes of the threads that met at the side's barrier, and
            // a write that has to cross NVLink and be acknowledged would hold every phase up by a round trip.
            while (s < a.n_steps) {
                PIPE_PHASE_BEGIN()
                asm volatile("barrier.sync 3, %0;" ::"r"(n_bar3) : "memory");
                const uint32_t n_all = min(sh.count[par], kPendP), n_send = min(n_all, kXPipeSeg);
                if (n_all > kXPipeSeg && lane == 0) atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
                const uint32_t xk = (a.seq0 + p) & 3u;
                for (uint32_t k = lane; k < n_send; k += 32u) {
                    const uint32_t ent = sh.pend[par][k];
                    for (uint32_t rk = 0; rk < a.n_ranks; ++rk)
                        if (rk != a.rank)
                            st_word(xp_ent(a.peers[rk] + a.xp_off, xk, a.rank, blockIdx.x, a.n_ranks, gridDim.x) + k, tag, ent);
                }
                __syncwarp();
                if (lane < a.n_ranks && lane != a.rank) st_word(xp_cnt(a.peers[lane] + a.xp_off, xk, a.rank, blockIdx.x), tag, n_send);
                // the list of this phase is written to the spike log and emptied one phase from now: not before this
                if (s + len < a.n_steps) asm volatile("barrier.arrive 4, 64;" ::: "memory");
                slot = (uint32_t)((slot + len) % S);
                s += len;
                ++p;
            }
            return;
        }
        while (s < a.n_steps) {
            PIPE_PHASE_BEGIN()
            const unsigned long long t_warp = a.profile ? gtimer() : 0ull;
            const uint32_t q = par ^ 1u;
            unsigned long long t_rows = 0ull;
            if (input_role) {
                // this phase's input spikes, from the start of the phase
                prepare_inputs(a, sh, L, tag, cc, start, slot, len, it, n_it, tot);
                // the spike log of the previous phase, while the update warps are still at work
                if (dwarp == log_warp && p > 0) {
                    // (the sender warp reads the same list: it has arrived here once it is done with it)
                    if (MULTI) asm volatile("barrier.sync 4, 64;" ::: "memory");
                    log_previous_phase(a, sh, lane, q, prev_start, log_pos, tot);
                }
                // has the other side finished already? (the leader has time to look: the update warps are still at work)
                // (only in phases of several steps: in one-step phases - the V1-scale network - the other side is never done
                // that early, and the look made this warp late for the update warps: 19.6 against 17.4 ms)
                if (it < 32u) early_look(sh, p, cnt_cons + (p & 3u), (p / 4u + 1u) * gridDim.x, s + len < a.n_steps, sync_dead || a.half < 2u);
                // then, once every update warp of the block has finished the phase, the block's own spikes
                asm volatile("barrier.sync 3, %0;" ::"r"(n_bar3) : "memory");
                queue_block_spikes(a, sh, L, tag, par, slot, it, n_it);
            } else {
                if (dtid == 0) sh.chunks[(p + 1u) % 3u] = 0u;   // the list of the NEXT phase was last read one phase ago
                if (p > 0) {
                    deliver_list(a, sh, sg, (p + 2u) % 3u, (uint32_t)prev_start + 1u, dwarp, lane, tot);
                    if (!multi) stage_flush(a, sg, lane);
                    if (multi) deliver_remote(a, sg, xp_self, (a.seq0 + p - 1u) & 3u, (uint32_t)prev_start + 1u, prev_slot, dwarp, kCW, lane, tot, sync_dead);
                }
                if (timer_d) t_rows = gtimer();
                if (IEXT && clamp_next) {
                    // changes effective from the next phase's first step: the update warps reload i_ext after
                    // they have seen this side finish
                    for (uint32_t g = cgi; g < a.ce_group_end && a.ce_group_step[g] <= start + len; ++g) {
                        const uint32_t b = a.ce_group_ptr[g], e = a.ce_group_ptr[g + 1];
                        for (uint32_t k = b + blockIdx.x * n_cons_threads + dtid; k < e; k += gridDim.x * n_cons_threads)
                            atomicAdd(&a.st.i_ext[a.ce_target[k] - a.lo], a.ce_delta[k]);
                    }
                }
            }
            // input warps belong to the producing side (their chunks go into this phase's lists); the chunk warps'
            // next phase - and their last pass after the loop - needs the producing side of this phase finished
            const unsigned long long t_work = timer_d ? gtimer() : 0ull;
            if (a.profile && lane == 0u) hist_add(a, input_role ? 1u : 2u, gtimer() - t_warp);
            if (input_role)
                prod_handover<MULTI>(a, sh, p, cnt_prod + (p & 3u), cnt_cons + (p & 3u), (p / 4u + 1u) * gridDim.x, n_prod_threads, it < 32u,
                                     sync_dead);
            else
                side_handover<MULTI>(a, cnt_cons + (p & 3u), cnt_prod + (p & 3u), (p / 4u + 1u) * gridDim.x, 1, n_cons_threads,
                              dwarp == 0u, true, sync_dead);
            if (timer_d) {
                const unsigned long long t_end = gtimer();
                acc_work += t_end - t_mark;   // the whole phase; acc_wait is the part spent in the hand-over
                acc_wait += t_end - t_work;
                acc_rows += (t_rows ? t_rows : t_mark) - t_mark;
                t_mark = t_end;
            }
            if (IEXT && clamp_next)
                while (cgi < a.ce_group_end && a.ce_group_step[cgi] <= start + len) ++cgi;
            prev_start = start;
            prev_slot = slot;
            slot = (uint32_t)((slot + len) % S);
            s += len;
            ++p;
        }
        // what the last phase emitted: delivered before the launch ends, so the ring is complete at rest
        if (p > 0) {
            if (!input_role) {
                deliver_list(a, sh, sg, (p + 2u) % 3u, (uint32_t)prev_start + 1u, dwarp, lane, tot);
                    if (!multi) stage_flush(a, sg, lane);
                if (multi) deliver_remote(a, sg, xp_self, (a.seq0 + p - 1u) & 3u, (uint32_t)prev_start + 1u, prev_slot, dwarp, kCW, lane, tot, sync_dead);
            }
            if (dwarp == log_warp) {
                const uint32_t q = (p & 1u) ^ 1u;
                const uint32_t n_rec = min(sh.count[q], kPendP);
                if (a.log_stamp && n_rec) write_log(a, sh, lane, n_rec, q, prev_start, log_pos);
                if (lane == 0) tot.spikes += n_rec;
            }
        }
        if (dwarp == log_warp && lane == 0 && a.log_stamp) {
            a.log_seg_cnt[blockIdx.x] = log_pos;
            if (log_pos > log_pos0) atomicAdd(&a.ctl->log_count, log_pos - log_pos0);
        }
        if (timer_d) {
            if (blockIdx.x == 0) {
                a.ctl->t_prop_ns += acc_work;
                a.ctl->t_sync2_ns += acc_wait;
                a.ctl->t_rows_ns += acc_rows;
                a.ctl->t_remote_wait_ns += tot.remote_wait_ns;
                a.ctl->t_remote_rows_ns += tot.remote_rows_ns;
            }
            if (a.blk_prof) {
                a.blk_prof[4 * blockIdx.x + 2] += acc_work - acc_wait;
                a.blk_prof[4 * blockIdx.x + 3] += acc_wait;
            }
        }
        if (tot.events) atomicAdd(&a.ctl->n_events, tot.events);
        if (tot.inputs) atomicAdd(&a.ctl->n_input_spikes, tot.inputs);
        if (tot.spikes) atomicAdd(&a.ctl->n_spikes, tot.spikes);
    }
#undef PIPE_PHASE_BEGIN
}

template <int BT>
static const void* pipelined_kernel_ptr_bt(bool has_theta, bool has_iext, bool multi) {
    if (multi)   // clamp changes are not supported with several ranks (the phase schedules would differ)
        return has_theta ? (const void*)pipelined_kernel<true, false, true, BT> : (const void*)pipelined_kernel<false, false, true, BT>;
    if (has_theta)
        return has_iext ? (const void*)pipelined_kernel<true, true, false, BT> : (const void*)pipelined_kernel<true, false, false, BT>;
    return has_iext ? (const void*)pipelined_kernel<false, true, false, BT> : (const void*)pipelined_kernel<false, false, false, BT>;
}

static const void* pipelined_kernel_ptr(bool has_theta, bool has_iext, bool multi, uint32_t block_warps) {
    return block_warps * 32u == (uint32_t)kBTSmall ? pipelined_kernel_ptr_bt<kBTSmall>(has_theta, has_iext, multi)
                                                   : pipelined_kernel_ptr_bt<kBT>(has_theta, has_iext, multi);
}

// Shared memory of a block: lists, type table, and a staging buffer of kStage chunks for each of `chunk_warps` warps
// (a small shared-memory carve-out leaves more L1 for the update warps' spilled registers).
size_t pipelined_smem(int n_types, uint32_t chunk_warps, uint32_t ring_stage_warps) {
    return sizeof(PipeShared) + type_table_bytes(n_types) +
           (size_t)chunk_warps * kStage * kChunk * sizeof(uint2) + (size_t)ring_stage_warps * 32 * 2 * kPorts * sizeof(float4);
}

uint32_t pipelined_max_update_warps() { return kMaxUpdWarps; }
uint32_t pipelined_warps() { return kWarps; }
uint32_t pipelined_warps_small() { return kBTSmall / 32; }

int pipelined_max_blocks(int device, bool has_theta, bool has_iext, size_t smem) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    for (uint32_t bw : {(uint32_t)kWarps, (uint32_t)(kBTSmall / 32)}) {
        int per_sm = 0;
        const void* f = pipelined_kernel_ptr(has_theta, has_iext, false, bw);
        if (cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, f, (int)bw * 32, smem) != cudaSuccess) return 0;
        if (per_sm <= 0) return 0;
    }
    return sms;   // one block per SM
}

cudaError_t launch_pipelined(const PersistArgs& a, bool has_theta, bool has_iext, int blocks, cudaStream_t s) {
    const size_t smem = pipelined_smem(a.n_types, a.block_warps - a.upd_warps - a.input_warps - (a.n_ranks > 1 ? 1u : 0u),
                                       a.ring_stage ? a.upd_warps : 0u);
    const void* f = pipelined_kernel_ptr(has_theta, has_iext, a.n_ranks > 1, a.block_warps);
    cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    PersistArgs copy = a;
    void* args[] = {&copy};
    return cudaLaunchCooperativeKernel(f, dim3(blocks), dim3(a.block_warps * 32u), args, smem, s);
}

}  // namespace bmtk
