// Shared device/host declarations of the bmtk_b200 engine (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bmtk_b200.h"

namespace bmtk {

constexpr int kPorts = BMTK_MAX_PORTS;
// A window spike-list entry packs (step inside the window, global source id).
constexpr int kStepBits = 5;
constexpr int kSrcBits = 32 - kStepBits;
constexpr uint32_t kSrcMask = (1u << kSrcBits) - 1u;
constexpr int kMaxWindow = 1 << kStepBits;

// Sticky device-side error bits (Ctl::error_flags).
enum : uint32_t {
    kErrSpikeListFull = 1u,
    kErrLogFull = 2u,
    kErrVirtListFull = 4u,
    kErrEventsFull = 8u,
    kErrExchangeTimeout = 16u,
    kErrSyncTimeout = 32u,
    kErrBadChunk = 64u,
};

// Per node type constants for one resolution, fp32 copies of fp64 host values.
// Unused ports and disabled mechanisms are neutral values so the update is branch-free:
// a port that does not exist has P11 = P21 = P31 = P32 = psc_init = 0; a type without
// after-spike currents has asc_coeff = asc_amps = 0 and asc_decay = asc_refr = 1.
// Members are grouped in 16-byte blocks so that the shared-memory copy is read with 128-bit loads.
struct __align__(16) TypeConsts {
    float P11[kPorts], P21[kPorts], P31[kPorts], P32[kPorts], psc_init[kPorts];
    float asc_decay[2], asc_coeff[2];
    float asc_refr[2], asc_amps[2];
    float P33, P30, th_inf, i_e;
    float v_reset, E_L, inv_G, delta_gain;   // delta_gain: 1 for iaf_psc_delta (ring input is a voltage jump), else 0
    float theta_spike_decay, theta_spike_refr, th_spike_add, reset_fraction;
    float reset_add, phi, abpara, theta_voltage_decay;
    int32_t n_ref;
    // bit0 spike-dependent threshold, bit1 adapting threshold, bit2 reset in the spike step
    // (iaf_psc_alpha), bit3 threshold test is >= (iaf_psc_alpha)
    int32_t flags;
    float asc_rec[2];   // asc_coeff / asc_decay: recovers the step mean the latest integrating step used from the current value
};
static_assert(sizeof(TypeConsts) % 16 == 0, "TypeConsts is copied word-wise and read with 128-bit loads");

// Device-resident control block: everything a replayed CUDA graph needs to find its place.
struct Ctl {
    unsigned long long step_base;   // absolute index of the first step of the current window
    unsigned long long n_events;    // synaptic events delivered so far
    unsigned long long n_spikes;    // neuron spikes so far
    unsigned long long n_input_spikes;
    uint32_t log_count;             // entries in the spike log since the last drain
    uint32_t error_flags;
    uint32_t ticket;                // blocks of the window-end kernel that have finished
    uint32_t sample_base;           // trace samples drained so far (absolute)
    uint32_t det_items;             // deterministic path: spike rows collected this window
    uint32_t det_events;            // deterministic path: events expanded this window
    uint32_t pad0, pad1;
    // persistent kernel, option "profile": device-timer totals of the two phases of every window
    unsigned long long t_update_ns, t_prop_ns, n_windows;
    unsigned long long t_sync1_ns, t_sync2_ns;   // of which: waiting in the two grid barriers (block 0's view)
    unsigned long long t_rows_ns;                // pipelined kernel: of the delivery warps' busy time, streaming rows
    unsigned long long t_remote_wait_ns;         // pipelined kernel, several ranks: of t_rows_ns, waiting for the other ranks' count words
    unsigned long long t_remote_rows_ns;         // ... and fetching + streaming the rows of their spikes
    unsigned long long pad2[1];
};

// Trial batching: T independent copies ("trials") of one network share its CSR. Cell c of trial t has
// index t*n_pad1 + c in every state array and ring plane (n_pad1 = cells per trial, padded to 4);
// Poisson cell v of trial t has source id n_cells_all + t*n_virtual + v and draws from its own Philox
// stream. With one trial n_cells_all = n_pad1 = n_global (ids are global neuron ids, trial 0).
struct IdSpace {
    uint32_t n_pad1, n_cells_all, n_virtual, n_global;
};
// source id -> CSR row and trial
__device__ __forceinline__ void split_source(const IdSpace& s, uint32_t id, uint32_t& row, uint32_t& trial) {
    if (id < s.n_cells_all) {
        trial = id / s.n_pad1;
        row = id - trial * s.n_pad1;
    } else {
        const uint32_t v = id - s.n_cells_all;
        trial = v / s.n_virtual;
        row = s.n_global + (v - trial * s.n_virtual);
    }
}

// Neuron state, structure of arrays; every array has n_pad entries (multiple of 4, 16-byte aligned).
struct StateSoA {
    float* U;        // membrane potential relative to E_L
    float* asc0;
    float* asc1;
    float* y1;       // [kPorts][n_pad]
    float* y2;       // [kPorts][n_pad]
    int32_t* refr;
    float* th_spike;    // nullptr unless a type uses it
    float* th_voltage;  // nullptr unless a type uses it
    float* i_ext;       // nullptr unless clamps exist
    const uint16_t* type;
};

struct UpdateArgs {
    StateSoA st;
    const TypeConsts* types;
    int32_t n_types;
    uint32_t n_local, n_pad;  // n_pad covers all trials
    uint32_t n_pad1;          // padded cells of ONE trial held here (= n_pad with one trial)
    IdSpace ids;
    uint32_t lo;              // global id of local neuron 0
    float* ring;              // [slots][kPorts][n_pad]
    uint32_t ring_slots;
    Ctl* ctl;
    uint32_t step_in_window;  // s: this launch executes step ctl->step_base + s
    uint32_t* send;           // [0] = count, then entries (s << kSrcBits | global id)
    uint32_t send_cap;
    uint32_t* log_stamp;      // spike log (nullptr = not recording)
    uint32_t* log_id;
    uint32_t log_cap;
    // on-line Poisson sources (nullptr = none)
    const uint4* poisson_thr; // per virtual source: CDF thresholds of k = 0..3
    uint32_t n_virtual, n_global, n_trials;
    uint32_t trial_base;      // Philox stream of local trial 0 (trials sharded over engines)
    uint64_t seed;
    uint32_t* virt;           // [0] = count, then entries, same packing as `send`
    uint32_t virt_cap;
};

struct PropArgs {
    const unsigned long long* rowptr;  // [n_rows + 1]
    const uint2* entries;              // {packed, weight bits}
    uint32_t target_bits;
    float* ring;
    uint32_t ring_slots, n_pad;
    uint32_t n_pad1;                   // local cells per trial (offset of a trial inside a ring plane)
    IdSpace ids;
    Ctl* ctl;
    // recurrent spikes: n_seg segments of seg_stride words, word 0 = count
    const uint32_t* gathered;
    uint32_t n_seg, seg_stride, seg_cap;
    // replayed virtual spikes: entries [in_ptr[step_base], in_ptr[step_base + window)) of (in_step, in_src)
    const uint32_t* in_ptr;            // indexed by absolute step - in_ptr_base, clamped
    unsigned long long in_ptr_base;
    uint32_t in_ptr_len;
    const uint32_t* in_step;
    const uint32_t* in_src;
    // on-line Poisson spikes of this window
    uint32_t* virt;
    uint32_t virt_cap;
    uint32_t window;                   // steps this window advanced
    uint32_t* send;                    // reset for the next window
};

// Launch wrappers (defined next to their kernels).
cudaError_t launch_glif_update(const UpdateArgs& a, bool has_theta, bool has_iext, cudaStream_t s);
cudaError_t launch_propagate_atomic(const PropArgs& a, cudaStream_t s);
int glif_update_blocks(uint32_t n_pad, uint32_t n_virtual);
cudaError_t launch_scatter_red_probe(float* cells, uint32_t n_cells, unsigned long long n_ops, cudaStream_t s);

}  // namespace bmtk
