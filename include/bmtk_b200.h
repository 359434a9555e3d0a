/*
 * bmtk_b200 C ABI — the B200 point-neuron engine that stands where BMTK PointNet calls NEST.
 *
 * The reference has no native FFI on this path: bmtk.simulator.pointnet talks to its engine
 * only through PyNEST calls. Each entry point below names the PyNEST call site(s) it replaces
 * (paths relative to the bmtk source tree). Host code binds these with ctypes
 * (bmtk_b200/_cabi.py).
 *
 * Conventions: every function returns 0 on success or a negative BMTK_E_* code;
 * bmtk_last_error() gives the message of the calling thread's last failure. Nothing throws
 * across the boundary and no device trap is ever raised on purpose. All pointers are HOST
 * pointers unless a parameter is named d_*; the engine copies what it needs. One engine per
 * GPU / per rank, driven by one host thread.
 */
#ifndef BMTK_B200_H
#define BMTK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define BMTK_MAX_PORTS 4

enum {
    BMTK_OK = 0,
    BMTK_E_INVALID = -1,    /* bad argument / call order */
    BMTK_E_CUDA = -2,       /* a CUDA call failed (message has the CUDA error string) */
    BMTK_E_OVERFLOW = -3,   /* a fixed-capacity device buffer (spike list, log, events) filled up */
    BMTK_E_UNSUPPORTED = -4,
    BMTK_E_COMM = -5,       /* NCCL unavailable or a collective failed */
    BMTK_E_DELAY = -6       /* a synaptic delay is shorter than one step */
};

/* NEST `glif_psc` parameters under their NEST names, as found in a NEST-format
 * dynamics_params file or produced by convert_aibs2nest
 * (bmtk/simulator/pointnet/glif_utils.py:259-418). Units: mV, pF, nS, ms, pA, 1/ms. */
typedef struct bmtk_glif_params {
    double V_m, V_th, g, E_L, C_m, t_ref, V_reset;
    double asc_init[2], asc_decay[2], asc_amps[2], asc_r[2];
    double tau_syn[BMTK_MAX_PORTS];
    double th_spike_add, th_spike_decay, voltage_reset_fraction, voltage_reset_add;
    double th_voltage_index, th_voltage_decay;
    int32_t n_ports;                    /* length of tau_syn in use, 1..BMTK_MAX_PORTS */
    int32_t spike_dependent_threshold;  /* "R" */
    int32_t after_spike_currents;       /* "ASC" */
    int32_t adapting_threshold;         /* "A" */
    double I_e;                         /* constant input current, pA */
    int32_t model;                      /* BMTK_MODEL_GLIF_PSC, _IAF_PSC_ALPHA or _IAF_PSC_DELTA */
    int32_t reserved;
} bmtk_glif_params;

/* `model` selects the conventions that differ between NEST models sharing these dynamics:
 * glif_psc holds V during refractoriness and resets when it ends, counts the refractory period
 * down in double precision and fires on V > V_th; iaf_psc_alpha (tau_syn = {tau_syn_ex,
 * tau_syn_in}, g = C_m / tau_m, no after-spike currents; the caller routes weights >= 0 to port 0
 * and weights < 0 to port 1) resets V in the spike step, is refractory for round(t_ref/dt) steps
 * and fires on V >= V_th. */
#define BMTK_MODEL_GLIF_PSC 0
#define BMTK_MODEL_IAF_PSC_ALPHA 1
/* NEST iaf_psc_delta (examples/point_120cells/network/cortex_node_types.csv:2-3): a weight is a jump of
 * the membrane potential in mV applied in the step the spike arrives; input that arrives while the
 * neuron is refractory is discarded; tau_syn and the receptor ports are unused (all ports add up). */
#define BMTK_MODEL_IAF_PSC_DELTA 2

typedef struct bmtk_engine bmtk_engine;

const char* bmtk_last_error(void);
/* Library version string, e.g. "bmtk_b200 0.1 sm_100a". */
const char* bmtk_version(void);

/* nest.ResetKernel + nest.SetKernelStatus({'resolution': dt, ...})
 * (bmtk/simulator/pointnet/pointsimulator.py:73-74). `device` is a CUDA ordinal. */
int bmtk_engine_create(bmtk_engine** out, int device, double dt_ms);
int bmtk_engine_destroy(bmtk_engine* e);

/* nest.Create(model, n, params), one call per node type
 * (bmtk/simulator/pointnet/sonata_adaptors.py:64-66, pointnetwork.py:144-159).
 * The network has n_global neurons with ids 0..n_global-1; this engine owns the contiguous
 * block [lo, lo+n_local). type_index[i] (i local) selects types[]. */
int bmtk_engine_set_nodes(bmtk_engine* e, uint64_t n_global, uint64_t lo, uint64_t n_local,
                          const uint16_t* type_index, int32_t n_types, const bmtk_glif_params* types);

/* nest.Create('spike_generator', n) for virtual cells (pointnetwork.py:187-216). Virtual cell v
 * is source id n_global + v in edge lists. */
int bmtk_engine_set_virtual(bmtk_engine* e, uint64_t n_virtual);

/* nest.Connect(srcs, trgs, 'one_to_one', syn_spec{weight[], delay[], receptor_type})
 * (pointnetwork.py:229-248; per-edge-type values from sonata_adaptors.py:268-357).
 * src: global source id (neuron or n_global+virtual); trg: global neuron id inside this engine's
 * block; weight in pA; delay in steps (>= 1, else BMTK_E_DELAY — the reference raises BadDelay,
 * pointnetwork.py:234-243); port 0-based (NEST receptor_type - 1). May be called several times
 * before finalize; edges accumulate in call order. */
int bmtk_engine_add_edges(bmtk_engine* e, uint64_t n_edges, const uint32_t* src, const uint32_t* trg,
                          const float* weight, const uint16_t* delay_steps, const uint8_t* port);

/* nest.SetStatus(spike_generator, {'spike_times': ...}) (pointnetwork.py:52-61). Spikes are given
 * as (virtual index, stamp in steps = ceil(t/dt) >= 1), any order. Replaces all stamps greater
 * than the current step; may be called between runs to stream inputs. */
int bmtk_engine_set_input_spikes(bmtk_engine* e, uint64_t n, const uint32_t* virt_index,
                                 const uint32_t* stamp_step);

/* On-line Poisson virtual cells (no counterpart in the reference, which only replays files made
 * by PoissonSpikeGenerator, bmtk/utils/reports/spike_trains/spike_trains.py:166-206): source v
 * fires k times in step n with k ~ Poisson(rate_hz[v]*dt), drawn from Philox4x32-10 with
 * counter (v, n) and key `seed`. rate_hz has n_virtual entries; rate*dt must be <= 0.25. */
int bmtk_engine_set_poisson(bmtk_engine* e, const float* rate_hz, uint64_t seed);

/* nest.Create('step_current_generator', {amplitude_times, amplitude_values}) + Connect with
 * delay = dt (bmtk/simulator/pointnet/modules/iclamp.py:42-54). Events: at the start of step
 * `step[i]` the external current of global neuron target[i] changes by delta_pA[i]. An amplitude
 * listed at time T becomes effective at step round(T/dt)+1. */
int bmtk_engine_set_clamp_events(bmtk_engine* e, uint64_t n, const uint64_t* step, const uint32_t* target,
                                 const float* delta_pA);

/* nest.Create('spike_recorder') + Connect(all gids, recorder)
 * (bmtk/simulator/pointnet/modules/record_spikes.py:134-136). */
int bmtk_engine_record_spikes(bmtk_engine* e, int enable);

/* nest.Create('multimeter', {'record_from': ['V_m'], 'interval': ...}) + Connect(mm, gids)
 * (bmtk/simulator/pointnet/modules/multimeter_reporter.py:103-115). ids are global neuron ids in
 * this engine's block; sample k (k >= 1) is V_m after the step that ends at k*interval. */
int bmtk_engine_record_vm(bmtk_engine* e, uint64_t n_ids, const uint32_t* ids, uint32_t interval_steps);

/* The same multimeter with other `record_from` names (multimeter_reporter.py:103-115 hands any name to NEST).
 * vars[n_vars] are BMTK_VAR_* codes, at most 8; record_vm is record_state with {BMTK_VAR_V_M}. A trace sample then
 * holds n_vars rows of n_ids values, [sample][variable][id], in the order of `vars`. I_syn is the sum of the ports'
 * post-synaptic currents (pA); ASCurrents_sum the step mean of the after-spike currents that the latest
 * integrating step used (it differs from NEST's held value in the one sample at which the refractory period ends);
 * threshold is V_th + spike + voltage component (mV, absolute). */
#define BMTK_VAR_V_M 0
#define BMTK_VAR_I_SYN 1
#define BMTK_VAR_ASC_SUM 2
#define BMTK_VAR_THRESHOLD 3
#define BMTK_VAR_TH_SPIKE 4
#define BMTK_VAR_TH_VOLTAGE 5
#define BMTK_VAR_I 6
int bmtk_engine_record_state(bmtk_engine* e, uint64_t n_ids, const uint32_t* ids, uint32_t interval_steps, int32_t n_vars,
                             const int32_t* vars);

/* Options (before finalize unless noted):
 *  "deterministic"  0|1  sorted segmented reduction instead of atomics in spike delivery
 *  "trials"         T >= 1 independent copies of the network that share the CSR (one rank, atomic
 *                   delivery, Poisson cells only): cell c of trial t is id t*n_pad1 + c in spike records,
 *                   probes and get_state (n_pad1 = counter "n_pad1" = n_local rounded up to 4), and Poisson
 *                   cell v of trial t draws from Philox counter (v, step, t)
 *  "trial_base"     Philox stream of local trial 0 (default 0), so that several engines can each take a
 *                   slice of one trial sweep
 *  "window"         steps per exchange window, 0 = min delay (default)
 *  "spike_capacity" entries of the per-window spike list, 0 = automatic
 *  "log_capacity"   entries of the device spike log between host drains
 *  "event_capacity" events per window the deterministic path can sort
 *  "persistent"     0|1 run each chunk as ONE cooperative kernel that loops over the steps with the
 *                   neuron state held in registers (default 1; single rank, atomic delivery; may
 *                   be changed between runs)
 *  "pipeline"       0|1 persistent stepping with update and delivery warps side by side on every SM, handing
 *                   over once per min_delay / 2 steps (default 1; used when the state fits in registers and the
 *                   minimum delay is at least 2 steps; counter "pipelined"; may be changed between runs)
 *  "pipeline_trials" with "trials" > 1: trials one launch of the pipelined kernel steps (a chunk of steps is run for
 *                   that many trials at a time, one group after the other, so that the ring slots a launch scatters
 *                   into stay in L2). Default 0: as many as the 12-warp block takes (else the 20-warp block) within
 *                   3/4 of L2; counter "pipeline_trials" has the value in use. Before finalize.
 *  "pipeline_warps" 0|12|20 warps of a block of the pipelined kernel. 12 warps have up to 168 registers a thread (no
 *                   spills in the update, packed fma.rn.f32x2 arithmetic) and are chosen (0, the default) where
 *                   they leave at least 5 warps to stream synapse chunks; else 20 warps at 96 registers.
 *  "tune"           pipelined kernel: 1 = scalar arithmetic, 2 = packed arithmetic in either block size (default 0:
 *                   packed in the 12-warp block only; same bits either way)
 *  "ring_stage"     0|1 pipelined kernel, minimum delay of 4 steps or more (phases of several steps): the ring cells of
 *                   the next step are copied to shared memory while a step computes (default 1; may be changed
 *                   between runs)
 *  "ring_prefetch"  0|1 persistent kernel with resident state: fetch the next step's ring slot into shared
 *                   memory with cp.async while the current step computes (default 0: on the 2-step
 *                   windows of the benchmark network it measured 3 % slower than plain L2 loads)
 *  "spike_store_reserve"  pin host memory for this many recorded spikes now (the store otherwise grows in
 *                   blocks of 2 Mi spikes as they arrive; any time)
 *  "phase_timers"   0|1 let the persistent kernels accumulate device time as seen by block 0 (counters
 *                   "phase_windows" = barrier-delimited phases timed; "phase_update_ns" / "phase_propagate_ns" =
 *                   time of the update / delivery side including its barrier wait, "phase_sync1_ns" /
 *                   "phase_sync2_ns" = that wait; the two sides follow each other in the two-phase kernel and
 *                   run side by side in the pipelined one, where "phase_rows_ns" is the row-streaming part)
 *  "use_graph"      0|1 replay each window as a CUDA graph when not persistent (default 1)
 *  "chunk_steps"    steps between host drains of the spike log / traces */
int bmtk_engine_set_option(bmtk_engine* e, const char* key, int64_t value);

/* Multi-GPU spike exchange: replaces NEST's MPI exchange inside nest.Simulate. uid is the
 * 128-byte ncclUniqueId made by bmtk_comm_unique_id on rank 0 and distributed by the caller;
 * libnccl is the path of the NCCL shared object to use (NULL = "libnccl.so.2"). A NULL uid creates no
 * communicator (for ranks that only use the peer-memory exchange below). */
int bmtk_comm_unique_id(void* uid128, const char* libnccl);
int bmtk_engine_comm_init(bmtk_engine* e, const void* uid128, int rank, int n_ranks, const char* libnccl);

/* Agreement of the ranks on the exchange layout (no counterpart in the reference: NEST's kernel
 * agrees on min_delay and its MPI buffer sizes internally when nest.Simulate prepares,
 * bmtk/simulator/pointnet/pointsimulator.py:166). A sender indexes the receiver's exchange buffer
 * with its own window, spike capacity and offsets, and the all-gather variant passes its own count to
 * the collective, so all ranks must derive these from the same numbers. Before finalize each rank
 * reads local_layout -> out4 = {minimum delay of its edges in steps (2^32-1 without edges), its
 * neurons, 1 if it has clamp events, 0}, the caller reduces (min, max, or) over the ranks by any means
 * and hands every rank the same in4 = {network minimum delay, largest block, any clamps, 0} with
 * set_global_layout. After finalize exchange_layout writes the 16-word description of what the rank's
 * buffer is laid out for (the same words sit at the head of the buffer); p2p_connect and
 * p2p_connect_pointers read every peer's words and finalize with an NCCL communicator all-gathers
 * them, and each returns BMTK_E_INVALID naming the differing quantity before any kernel runs.
 * exchange_layout_compare is that comparison as a host function. */
int bmtk_engine_local_layout(bmtk_engine* e, uint64_t* out4);
int bmtk_engine_set_global_layout(bmtk_engine* e, const uint64_t* in4);
int bmtk_engine_exchange_layout(bmtk_engine* e, uint64_t* out16);
int bmtk_exchange_layout_compare(const uint64_t* mine16, const uint64_t* theirs16, int their_rank);

/* Spike exchange inside the stepping kernel, over peer memory (NVLink / NVSwitch) instead of one
 * NCCL all-gather per window: after finalize every rank exports the handle of its exchange buffer
 * (a 64-byte cudaIpcMemHandle_t), the caller distributes the handles, and p2p_connect maps all
 * n_ranks of them (handles = n_ranks x 64 bytes, in rank order). From then on the persistent kernel
 * of every rank stores its window's spike ids straight into every rank's inbox and waits, with a
 * bound of about one second, for the other ranks' windows; a time-out ends the run with
 * BMTK_E_COMM. Ranks are separate processes on separate GPUs and must call run() with the same
 * step counts. Without p2p_connect several ranks use the per-step kernels and NCCL. */
int bmtk_engine_p2p_handle(bmtk_engine* e, void* handle64);
int bmtk_engine_p2p_connect(bmtk_engine* e, const void* handles);
/* The same for ranks that live in ONE process (one engine per GPU, peer access enabled by the
 * caller): p2p_buffer returns the device pointer of an engine's exchange buffer, and
 * p2p_connect_pointers takes the n_ranks pointers in rank order. comm_init may then be given a
 * NULL id (no NCCL communicator is created). */
int bmtk_engine_p2p_buffer(bmtk_engine* e, void** d_buffer);
int bmtk_engine_p2p_connect_pointers(bmtk_engine* e, void* const* d_buffers);

/* Builds the delay-bucketed CSR on the device, allocates state and ring buffers, initialises
 * V = V_m, ASC = asc_init. Must precede run. */
int bmtk_engine_finalize(bmtk_engine* e);

/* nest.Simulate(n_steps*dt) (bmtk/simulator/pointnet/pointsimulator.py:166). */
int bmtk_engine_run(bmtk_engine* e, uint64_t n_steps);

/* Recorder read-out (record_spikes.py:138-161 / multimeter_reporter.py:117-167 read NEST's .dat
 * files instead). Spikes are returned sorted by (stamp, id); stamp is in steps (time = stamp*dt),
 * id is the global neuron id. Fetching drains the host-side store. */
int bmtk_engine_spike_count(bmtk_engine* e, uint64_t* n);
int bmtk_engine_fetch_spikes(bmtk_engine* e, uint64_t cap, uint32_t* stamp_step, uint32_t* id, uint64_t* n_out);
int bmtk_engine_trace_samples(bmtk_engine* e, uint64_t* n_samples);
int bmtk_engine_fetch_trace(bmtk_engine* e, uint64_t cap_samples, float* vm /* [samples][n_ids] */,
                            uint64_t* n_out);

/* State read-out for tests/checkpoints: var in {"V_m","U","asc0","asc1","y1_0".."y1_3","y2_0".."y2_3",
 * "i_ext","th_spike","th_voltage"}; out has n_local floats. "refr" returns the counter as float. */
int bmtk_engine_get_state(bmtk_engine* e, const char* var, float* out);

/* CSR read-out for bit-exact checks against an independent build. rowptr has n_rows+1 entries;
 * packed[k] = delay << (target_bits+2) | port << target_bits | local_target. Pass NULL to query
 * sizes only. */
int bmtk_engine_csr_info(bmtk_engine* e, uint64_t* n_rows, uint64_t* n_edges, uint32_t* target_bits,
                         uint32_t* max_delay, uint32_t* min_delay, uint32_t* ring_slots);
int bmtk_engine_get_csr(bmtk_engine* e, uint64_t* rowptr, uint32_t* packed, float* weight);

/* Counters: "events" (synaptic events delivered), "spikes" (neuron spikes), "steps",
 * "launches" (kernels launched by run), "update_ns"/"propagate_ns" (device time when
 * option "profile" is 1), "window". */
int bmtk_engine_get_counter(bmtk_engine* e, const char* name, uint64_t* out);

/* The delivery step of nest.Simulate on its own (event delivery into the targets' ring buffers,
 * bmtk/simulator/pointnet/pointsimulator.py:166), for callers that keep the CSR and the ring
 * buffer in their own device memory. All d_* are DEVICE pointers: d_rowptr[n_rows+1],
 * d_entries[E] as {uint32 packed, float weight} pairs in the layout of bmtk_engine_get_csr,
 * the spikes as (source row, emitting step) pairs, d_ring[ring_slots][4][n_pad]. Every listed
 * spike adds its row's weights to ring[(step + delay) mod ring_slots][port][target].
 * deterministic = 1 sums in a fixed order (sorted segmented reduction), 0 uses atomics.
 * Allocates and frees its workspace with cudaMalloc on every call; returns after the stream
 * has finished. `stream` is a cudaStream_t (NULL = default stream). */
int bmtk_propagate_spikes(const uint64_t* d_rowptr, const void* d_entries, uint32_t target_bits,
                          uint32_t n_spikes, const uint32_t* d_spike_src, const uint32_t* d_spike_step,
                          float* d_ring, uint32_t ring_slots, uint32_t n_pad, int deterministic, void* stream);

/* The same deterministic delivery as bmtk_propagate_spikes(..., deterministic = 1, ...), for
 * callers that must not allocate device memory when they call it. (No counterpart in the
 * reference, which leaves all memory management to NEST.) Such callers exist: a plugin living
 * inside a host application's fixed memory pool, a latency-bound loop that may not take the
 * allocator's locks, a process whose network already fills the GPU. This entry point calls no
 * cudaMalloc/cudaFree and no allocating library routine; its scratch is a fixed array of about
 * 8.3 MB built into the library, which every GPU that loads the library holds until exit.
 * Limits per call: at most 4096 spikes and 262 144 synaptic events (sum of the listed rows'
 * lengths); a longer spike list is refused with BMTK_E_INVALID, more events with
 * BMTK_E_OVERFLOW, in both cases before the ring is touched (the event total is formed in 64 bits,
 * so repeated listings of long rows cannot wrap it into range).
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call before starting any stream capture. `stream` must belong to the device
 * that is current when the call is made: the scratch used is the current device's copy. All calls share the one array and it
 * keeps the previous call's contents (the entry point re-initialises what it needs), so two calls
 * whose GPU work could overlap - different streams, different host threads - race; serialise them.
 * Inputs and outputs are the caller's device memory exactly as for bmtk_propagate_spikes; the
 * call returns after the stream has finished. */
int bmtk_propagate_spikes_noalloc(const uint64_t* d_rowptr, const void* d_entries, uint32_t target_bits,
                                  uint32_t n_spikes, const uint32_t* d_spike_src, const uint32_t* d_spike_step,
                                  float* d_ring, uint32_t ring_slots, uint32_t n_pad, void* stream);

/* Checkpoint / resume (the reference has none; its block_run keys are dead code,
 * bmtk/simulator/pointnet/pointsimulator.py:118-132,215-218). save_state writes the step counter, the
 * neuron state arrays and the ring buffer of this engine to a file; load_state restores them into an
 * engine that was built and finalized from the same network, partition and dt. Recorder stores are
 * emptied by a load; replayed input spikes must be handed over again after it. */
int bmtk_engine_save_state(bmtk_engine* e, const char* path);
int bmtk_engine_load_state(bmtk_engine* e, const char* path);

/* Measures the device's rate of scattered fp32 reductions (no counterpart in the reference): n_ops
 * `red.global.add.f32` into pseudo-random cells of a zeroed buffer of n_cells floats, `repeats` times,
 * timed with CUDA events. This is the ceiling of any delivery that ends in one reduction per synaptic
 * event; bench and microbench report the delivery kernels against it. */
int bmtk_probe_scatter_reductions(int device, uint64_t n_cells, uint64_t n_ops, int repeats, double* ms_per_pass);

/* One-way latency of the spike exchange's primitive between two connected ranks (no counterpart in the reference): a
 * single thread on each of the two GPUs bounces a tagged 8-byte word `rounds` times with a plain peer store and a
 * polling load, as the stepping kernels do. Both ranks call it at the same time, one with initiator = 1 and one with
 * initiator = 0, each naming the other as peer_rank; one_way_ns receives half the mean round trip (meaningful on the
 * initiator). Every wait is bounded (a few seconds), after which the call returns BMTK_E_COMM. A phase of the
 * stepping kernel with several ranks cannot be shorter than this latency plus the work that depends on it. */
int bmtk_engine_p2p_pingpong(bmtk_engine* e, int peer_rank, int initiator, uint32_t rounds, double* one_way_ns);

/* Per-block phase profile of the pipelined stepping kernel (no counterpart in the reference). With option
 * phase_timers = 1 every block sums, with the device timer, how long its producing side (update and input warps)
 * and its delivering side (chunk warps) were busy and how long each waited in the hand-over at the end of a phase.
 * out4 receives 4 values per block {producing busy, producing wait, delivering busy, delivering wait} in ns since
 * the last call and the sums are cleared; n_blocks receives the block count (0 when the kernel is not in use; pass
 * out4 = NULL to ask for it). Behind the blocks' values follow five histograms of 32 bins of 250 ns (160 values): how
 * long after the start of a phase a warp reached the hand-over, for update, input and chunk warps, and how long after it
 * an update warp had finished its last step, for warps without and with a spike; cap_blocks must therefore be at least
 * n_blocks + 40. Shows whether a phase is long because one block is slow or because the hand-over is. */
int bmtk_engine_block_profile(bmtk_engine* e, uint64_t cap_blocks, uint64_t* out4, uint64_t* n_blocks);

/* Synthetic network generator on the device: the stand-in for bmtk.builder on this path (the reference builds its
 * example networks on the host with per-pair connection rules, examples/point_450glifs/build_network.py, and writes
 * them with bmtk/builder/network_adaptors/dm_network.py:103-121). Samples the incoming edges of the target neurons
 * [lo, hi) of a distance-dependent network: per target a number of candidates with mean lambda[target type]; each
 * candidate picks a source class with odds q_exc : q_inh, a Gaussian displacement of sigma[class][target type] taken
 * from the 4096-quantile table gauss_table, the grid cell (side 1 / inv_cell, grid x grid cells over the square
 * around the disk of `radius`) it lands in, is kept with probability cell_count / cell_max and given to a uniformly
 * chosen neuron cell_ids[class][cell_start + i] of the cell; weight = w_base[source type][target type] x
 * lognorm_table[.] (x -inh_scale for inhibitory sources), delay uniform in [delay_min_ms, delay_max_ms] rounded to
 * dt steps, port = (source inhibitory) + 2 (target inhibitory). Randomness: Philox4x32-10, counters
 * (target, candidate, 0 | 1, 0), key = seed; arithmetic is single IEEE operations in a fixed order, so the edge list is
 * a pure function of the specification (independent of the partition into [lo, hi) blocks and of the device).
 * Edges come out ordered by (target, candidate). Call with cap = 0 and src = NULL for the count, then with arrays of
 * at least that many entries (host memory). All pointers in the specification are HOST arrays. */
typedef struct bmtk_gen_spec {
    uint32_t n_neurons, n_types, lo, hi;
    const uint16_t* type_index;        /* [n_neurons] */
    const uint8_t* type_is_inh;        /* [n_types] */
    const float *x, *y;                /* [n_neurons] positions, um */
    const float* sigma;                /* [2][n_types]: (source class, target type), um */
    const float* w_base;               /* [n_types][n_types]: (source type, target type), pA */
    const float *q_exc, *q_inh;        /* [n_types]: odds of an excitatory / inhibitory source by target type */
    const float* lambda;               /* [n_types]: mean number of candidates per target */
    const float *gauss_table, *lognorm_table;   /* [4096] each */
    const uint32_t* cell_start[2];     /* [grid*grid] per source class */
    const uint32_t* cell_count[2];
    const uint32_t* cell_ids[2];       /* [class_size] neuron ids sorted by cell */
    uint32_t class_size[2];
    float cell_max[2];                 /* largest cell_count of the class */
    uint32_t grid;
    float radius, inv_cell, inh_scale, delay_min_ms, delay_max_ms, dt;
    uint64_t seed;
} bmtk_gen_spec;
int bmtk_generate_distance_edges(const bmtk_gen_spec* spec, int device, uint64_t cap, uint32_t* src, uint32_t* trg, float* weight,
                                 uint16_t* delay_steps, uint8_t* port, uint64_t* n_edges);

/* Device-side timing of the engine's own stream (no counterpart in the reference): mark records a
 * CUDA event in one of 8 slots after everything enqueued so far; elapsed_ms waits for `to_slot`
 * and returns the device time between two marks. */
int bmtk_engine_mark(bmtk_engine* e, int slot);
int bmtk_engine_elapsed_ms(bmtk_engine* e, int from_slot, int to_slot, double* ms);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* BMTK_B200_H */
