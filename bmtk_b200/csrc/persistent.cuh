#pragma once
#include "common.cuh"
#ifdef __CUDACC__
#include "glif_math.cuh"
#endif

namespace bmtk {

constexpr uint32_t kXRanks = 16;   // most ranks an exchange buffer is laid out for

// Arguments of one persistent launch (a chunk of steps on one GPU).
struct PersistArgs {
    // neurons
    StateSoA st;
    const TypeConsts* types;
    int32_t n_types;
    uint32_t n_local, n_pad, lo, n_global;
    uint32_t n_pad1, n_trials;   // cells per trial (padded) and number of trials sharing the CSR
    uint32_t trial_base;         // Philox stream of local trial 0
    IdSpace ids;
    float* ring;
    uint32_t ring_slots;
    Ctl* ctl;
    // Window spike lists, double buffered by window parity. An entry is {step_in_window << kSrcBits |
    // source, row length, row begin lo, row begin hi}; list_counts[parity] is its fill. Blocks collect
    // their spikes in shared memory and append them with one atomic per block per window.
    uint4* lists[2];
    uint32_t* list_counts;     // [2]
    uint32_t send_cap;
    uint32_t* log_stamp;       // spike log (nullptr = not recording), fill in ctl->log_count
    uint32_t* log_id;
    uint32_t log_cap;
    // on-line Poisson cells
    const uint4* poisson_thr;
    uint32_t n_virtual;
    uint64_t seed;
    uint32_t* virts[2];
    uint32_t virt_cap;
    // CSR and replayed inputs
    const unsigned long long* rowptr;
    const uint2* entries;
    uint32_t target_bits;
    const uint32_t* in_ptr;
    unsigned long long in_ptr_base;
    uint32_t in_ptr_len;
    const uint32_t* in_step;
    const uint32_t* in_src;
    // stepping
    uint32_t n_steps, window;
    uint32_t half;             // pipelined kernel: steps per phase, <= min_delay / 2
    // pipelined kernel: chunk lists [3][blocks][pipe_seg_cap] of {first entry, length, ring slot, phase tag}
    uint4* pipe_seg;
    uint32_t pipe_seg_cap;
    unsigned long long n_entries;   // CSR entries (bounds of a chunk descriptor)
    uint32_t* pipe_sync;       // pipelined kernel: [0..3] blocks whose producing side, [4..7] whose chunk warps finished phase p mod 4
    uint32_t log_seg_cap;      // pipelined kernel: block b logs spikes into [b * log_seg_cap, (b + 1) * log_seg_cap) ...
    uint32_t* log_seg_cnt;     // ... and leaves its entry count here
    uint32_t block_warps;      // pipelined kernel: warps of a block (20, or 12 where that leaves enough chunk warps)
    uint32_t upd_warps;        // pipelined kernel: update warps of a block
    // pipelined kernel, several trials: one launch steps the cells [cell0, cell0 + n_cells) - whole trials, the first of
    // them trial0 - so that their ring slots stay in L2; the launches of a chunk of steps follow one another over the
    // trials, append to the same spike log (log_append) and only the last moves the clock (advance_clock)
    uint32_t cell0, n_cells, trial0, log_append, advance_clock;
    uint32_t ring_stage;       // pipelined kernel, phases of several steps: copy the next step's ring cells to shared memory ahead
    uint32_t input_warps;      // pipelined kernel: warps of a block that prepare input spikes; the rest stream chunks
    // clamp events grouped by step: group g covers events [ce_group_ptr[g], ce_group_ptr[g+1])
    const unsigned long long* ce_group_step;
    const uint32_t* ce_group_ptr;
    uint32_t ce_group_begin, ce_group_end;
    const uint32_t* ce_target;
    const float* ce_delta;
    // V_m probes: probe_slot[i] = trace column of local neuron i or -1
    const int32_t* probe_slot;
    uint32_t n_probe, probe_interval;
    uint32_t n_probe_vars, probe_vars;   // recorded variables: count and their BMTK_VAR_* codes, 4 bits each; a trace
                                         // sample is [variable][probe]
    float* trace;
    uint32_t trace_cap;
    uint32_t profile;
    uint32_t ring_prefetch;    // RESIDENT: copy the next step's ring slot to shared memory while this step computes
    unsigned long long* blk_prof;   // pipelined kernel, option phase_timers: per block {producing side busy ns, its hand-over wait ns,
                               // delivering side busy ns, its hand-over wait ns}, summed over the launch
    uint32_t tune;             // pipelined kernel: 1 = scalar arithmetic in every block size, 2 = packed in every block size
    // Spike exchange between ranks over peer memory (n_ranks > 1). Every rank owns an exchange
    // buffer of 64-bit words laid out as  counts[2][kXRanks] | inbox[2][n_ranks][xchg_cap];
    // peers[r] is rank r's buffer as mapped into this process (peers[rank] is the local one).
    // Every word is {window sequence number : 32 | payload : 32} written with ONE 8-byte store, so a
    // reader knows a word belongs to the window it is waiting for by its tag alone and no
    // system-wide fence is needed (the payload of a count word is the number of spikes, of an inbox
    // word a spike entry). Window `seq` uses parity seq & 1; rank r stores its spikes of the window
    // into inbox[parity][r] of EVERY rank and then its count into counts[parity][r] of every rank.
    uint32_t n_ranks, rank;
    unsigned long long* peers[kXRanks];
    uint32_t xchg_cap;
    uint32_t seq0;             // windows completed before this launch
    uint32_t xp_off;           // pipelined kernel: where its exchange area starts in an exchange buffer (64-bit words)
};

#ifdef __CUDACC__
// ---- device helpers shared by the persistent kernels

// ring cells and lists are written by other SMs between barriers: read them through L2
__device__ __forceinline__ F4 ld4cg(const float* p) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(p));
    return F4{{t.x, t.y, t.z, t.w}};
}

__device__ __forceinline__ unsigned long long gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

typedef unsigned long long u64;

// exchange words: {sequence number : 32 | payload : 32}, one 8-byte store / load each
__device__ __forceinline__ void st_word(u64* p, uint32_t seq, uint32_t payload) {
    *reinterpret_cast<volatile u64*>(p) = ((u64)seq << 32) | payload;
}
__device__ __forceinline__ u64 ld_word(const u64* p) { return *reinterpret_cast<const volatile u64*>(p); }

// bound of every wait on a peer: x (load + 100 ns sleep), about a second
constexpr unsigned int kWaitSpins = 4000000u;
#endif

constexpr size_t xchg_words(uint32_t n_ranks, uint32_t cap) { return 2 * (size_t)kXRanks + 2 * (size_t)n_ranks * cap; }

// Exchange area of the pipelined kernel, in 64-bit words {phase tag : 32 | payload : 32} like the
// two-phase area, behind it in every rank's exchange buffer:
//   cnt[4][kXRanks][kXBlocks] | ent[4][n_ranks][blocks][kXPipeSeg]
// cnt / ent hold what block b of rank r emitted in the phase with index p mod 4 (count; entries
// step_in_phase << kSrcBits | global id), written by the emitting rank with plain 8-byte peer stores.
// A word is valid when its tag is the phase's (first step + 1, the same on every rank), so no fence
// and no counter crosses the link: block b of a rank waits for the count word of block b of every
// other rank, and for each entry's tag.
constexpr uint32_t kXBlocks = 512;
constexpr uint32_t kXPipeSeg = 256;   // spikes one block can send in one phase
constexpr size_t xpipe_words(uint32_t n_ranks, uint32_t blocks) {
    return 4 * (size_t)kXRanks * kXBlocks + 4 * (size_t)n_ranks * blocks * kXPipeSeg;
}
#ifdef __CUDACC__
__device__ __forceinline__ u64* xp_cnt(u64* xp, uint32_t k, uint32_t r, uint32_t b) {
    return xp + ((size_t)k * kXRanks + r) * kXBlocks + b;
}
__device__ __forceinline__ u64* xp_ent(u64* xp, uint32_t k, uint32_t r, uint32_t b, uint32_t n_ranks, uint32_t blocks) {
    return xp + 4 * (size_t)kXRanks * kXBlocks + (((size_t)k * n_ranks + r) * blocks + b) * kXPipeSeg;
}
#endif

const void* persistent_kernel_ptr(bool has_theta, bool has_iext, bool resident);
int persistent_max_blocks(int device, bool has_theta, bool has_iext, bool resident, size_t smem);
uint32_t persistent_threads_per_block();
size_t persistent_smem(int n_types);
cudaError_t launch_persistent(const PersistArgs& a, bool has_theta, bool has_iext, bool resident, int blocks,
                              cudaStream_t s);

}  // namespace bmtk
