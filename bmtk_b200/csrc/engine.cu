// Engine object and C ABI of bmtk_b200: owns device memory, builds the CSR, drives the
// per-window kernel sequence (w x glif_update [+ snapshot] -> [all-gather] -> propagate) on one
// stream, replays it as a CUDA graph, drains the spike log and traces to the host in chunks.
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "csr_build.cuh"
#include <chrono>
#include <cstddef>

#include "persistent.cuh"
#include "pipeline.cuh"
#include "propagate_det.cuh"

namespace bmtk {

thread_local std::string g_last_error;

static int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define CU(x)                                                                                     \
    do {                                                                                          \
        cudaError_t e_ = (x);                                                                     \
        if (e_ != cudaSuccess)                                                                    \
            return fail(BMTK_E_CUDA, "%s failed: %s (%s:%d)", #x, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

// ---------------------------------------------------------------------------------------------
// Per-type constants (fp64 on the host, stored fp32): exact-integration propagators of the
// linear sub-threshold system for one resolution h.

// x + expm1(-x) without cancellation for small |x|.
static double cross_term(double x) {
    if (std::fabs(x) < 1e-3)
        return x * x * (0.5 + x * (-1.0 / 6.0 + x * (1.0 / 24.0 + x * (-1.0 / 120.0 + x / 720.0))));
    return x + std::expm1(-x);
}

static int compute_type_consts(const bmtk_glif_params& p, double h, TypeConsts& c) {
    if (!(p.C_m > 0) || !(p.g > 0)) return fail(BMTK_E_INVALID, "C_m and g must be positive");
    if (!(p.t_ref > 0) && p.model == BMTK_MODEL_GLIF_PSC) return fail(BMTK_E_INVALID, "t_ref must be positive");
    if (p.n_ports < 1 || p.n_ports > kPorts) return fail(BMTK_E_INVALID, "n_ports must be 1..%d", kPorts);
    std::memset(&c, 0, sizeof(c));
    const double tau = p.C_m / p.g;
    c.P33 = (float)std::exp(-h / tau);
    c.P30 = (float)(-std::expm1(-h / tau) / p.g);
    const bool delta = p.model == BMTK_MODEL_IAF_PSC_DELTA;
    c.delta_gain = delta ? 1.f : 0.f;
    for (int k = 0; k < (delta ? 0 : p.n_ports); ++k) {
        const double ts = p.tau_syn[k];
        if (!(ts > 0)) return fail(BMTK_E_INVALID, "tau_syn must be positive");
        const double a = 1.0 / ts, b = 1.0 / tau, d = b - a, x = d * h;
        const double ea = std::exp(-a * h);
        c.P11[k] = (float)ea;
        c.P21[k] = (float)(h * ea);
        c.psc_init[k] = (float)(std::exp(1.0) / ts);
        if (x == 0.0) {
            c.P32[k] = (float)(h * std::exp(-b * h) / p.C_m);
            c.P31[k] = (float)(0.5 * h * h * std::exp(-b * h) / p.C_m);
        } else {
            c.P32[k] = (float)(ea * (-std::expm1(-x)) / (d * p.C_m));
            c.P31[k] = (float)(ea * cross_term(x) / (d * d * p.C_m));
        }
    }
    for (int j = 0; j < 2; ++j) {
        if (p.after_spike_currents) {
            const double k = p.asc_decay[j];
            if (!(k > 0)) return fail(BMTK_E_INVALID, "asc_decay must be positive");
            c.asc_decay[j] = (float)std::exp(-k * h);
            c.asc_coeff[j] = (float)(-std::expm1(-k * h) / (k * h));
            c.asc_refr[j] = (float)(p.asc_r[j] * std::exp(-k * p.t_ref));
            c.asc_amps[j] = (float)p.asc_amps[j];
            c.asc_rec[j] = (float)(-std::expm1(-k * h) / (k * h) / std::exp(-k * h));
        } else {
            c.asc_decay[j] = 1.f;
            c.asc_coeff[j] = 0.f;
            c.asc_refr[j] = 1.f;
            c.asc_amps[j] = 0.f;
        }
    }
    c.th_inf = (float)(p.V_th - p.E_L);
    c.v_reset = (float)(p.V_reset - p.E_L);
    c.E_L = (float)p.E_L;
    // NEST counts the refractory period down in double precision, h per step, until <= 0.
    double r = p.t_ref;
    int n = 0;
    do {
        r -= h;
        ++n;
    } while (r > 0.0 && n < (1 << 30));
    c.n_ref = n;
    c.flags = (p.spike_dependent_threshold ? 1 : 0) | (p.adapting_threshold ? 2 : 0);
    c.i_e = (float)p.I_e;
    if (p.model == BMTK_MODEL_IAF_PSC_ALPHA || p.model == BMTK_MODEL_IAF_PSC_DELTA) {
        if (p.spike_dependent_threshold || p.adapting_threshold || p.after_spike_currents)
            return fail(BMTK_E_INVALID, "iaf_psc_alpha / iaf_psc_delta have no threshold dynamics or after-spike currents");
        c.flags |= 4 | 8;
        c.n_ref = (int)std::llround(p.t_ref / h);
        if (c.n_ref < 1) c.n_ref = 1;  // a spike always costs the step it happens in
    } else if (p.model != BMTK_MODEL_GLIF_PSC) {
        return fail(BMTK_E_INVALID, "unknown model %d", p.model);
    }
    c.theta_spike_decay = (float)std::exp(-p.th_spike_decay * h);
    c.theta_spike_refr = (float)std::exp(-p.th_spike_decay * p.t_ref);
    c.th_spike_add = (float)p.th_spike_add;
    c.reset_fraction = (float)p.voltage_reset_fraction;
    c.reset_add = (float)p.voltage_reset_add;
    c.inv_G = (float)(1.0 / p.g);
    if (p.adapting_threshold) {
        c.theta_voltage_decay = (float)std::exp(-p.th_voltage_decay * h);
        c.phi = (float)(p.th_voltage_index / (p.th_voltage_decay - p.g / p.C_m));
        c.abpara = (float)(p.th_voltage_index / p.th_voltage_decay);
    }
    return BMTK_OK;
}

// ---------------------------------------------------------------------------------------------
// Small kernels owned by the engine.

__global__ void init_state_kernel(StateSoA st, const TypeConsts* types, const float* init /*[n_types][3]*/,
                                  uint32_t n_pad) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    const uint16_t t = st.type[i];
    st.U[i] = init[t * 3 + 0];
    st.asc0[i] = init[t * 3 + 1];
    st.asc1[i] = init[t * 3 + 2];
    for (int p = 0; p < kPorts; ++p) {
        st.y1[(size_t)p * n_pad + i] = 0.f;
        st.y2[(size_t)p * n_pad + i] = 0.f;
    }
    st.refr[i] = 0;
    if (st.th_spike) st.th_spike[i] = 0.f;
    if (st.th_voltage) st.th_voltage[i] = 0.f;
    if (st.i_ext) st.i_ext[i] = 0.f;
}

// Clamp events [b, e): i_ext[target - lo] += delta. Events of one step may repeat a target.
__global__ void apply_clamp_kernel(float* i_ext, const uint32_t* target, const float* delta, uint32_t b, uint32_t e,
                                   uint32_t lo) {
    const uint32_t k = b + blockIdx.x * blockDim.x + threadIdx.x;
    if (k < e) atomicAdd(&i_ext[target[k] - lo], delta[k]);
}

// V_m probe: after the step that ends at a multiple of `interval`, writes V_m = U + E_L of the
// probed neurons into trace[sample][q].
__global__ void snapshot_kernel(Ctl* ctl, uint32_t step_in_window, uint32_t interval, const uint32_t* ids,
                                uint32_t n_ids, StateSoA st, uint32_t n_pad, const TypeConsts* types,
                                float* trace, uint32_t cap_samples, uint32_t n_vars, uint32_t vars) {
    const unsigned long long done = ctl->step_base + step_in_window + 1ull;
    if (done % interval) return;
    const unsigned long long sample = done / interval - 1ull - ctl->sample_base;
    if (sample >= cap_samples) return;  // the host sizes chunks so that this cannot happen
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t q = blockIdx.x * blockDim.x + threadIdx.x; q < n_ids; q += stride) {
        const uint32_t i = ids[q];
        const TypeConsts& c = types[st.type[i]];
        for (uint32_t v = 0; v < n_vars; ++v) {
            float x;
            switch ((vars >> (4u * v)) & 15u) {   // the same expressions as Neuron4::probe_value
                case BMTK_VAR_I_SYN:
                    x = __fadd_rn(__fadd_rn(__fadd_rn(st.y2[i], st.y2[(size_t)n_pad + i]), st.y2[2 * (size_t)n_pad + i]), st.y2[3 * (size_t)n_pad + i]);
                    break;
                case BMTK_VAR_ASC_SUM: x = __fmaf_rn(c.asc_rec[0], st.asc0[i], __fmul_rn(c.asc_rec[1], st.asc1[i])); break;
                case BMTK_VAR_THRESHOLD:
                    x = __fadd_rn(__fadd_rn(__fadd_rn(c.th_inf, st.th_spike ? st.th_spike[i] : 0.f), st.th_voltage ? st.th_voltage[i] : 0.f), c.E_L);
                    break;
                case BMTK_VAR_TH_SPIKE: x = st.th_spike ? st.th_spike[i] : 0.f; break;
                case BMTK_VAR_TH_VOLTAGE: x = st.th_voltage ? st.th_voltage[i] : 0.f; break;
                case BMTK_VAR_I: x = __fadd_rn(st.i_ext ? st.i_ext[i] : 0.f, c.i_e); break;
                default: x = __fadd_rn(st.U[i], c.E_L);
            }
            trace[((size_t)sample * n_vars + v) * n_ids + q] = x;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// NCCL through dlopen: the library has no link-time dependency on it.

struct Uid {
    char internal[128];
};
struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, /*ncclUniqueId by value*/ Uid, int) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;

static int load_nccl(const char* path) {
    if (g_nccl.handle) return BMTK_OK;
    const char* p = path && path[0] ? path : "libnccl.so.2";
    void* h = dlopen(p, RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(BMTK_E_COMM, "cannot load NCCL from '%s': %s", p, dlerror());
    g_nccl.GetUniqueId = (int (*)(void*))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(void**, int, Uid, int))dlsym(h, "ncclCommInitRank");
    g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(h, "ncclAllGather");
    g_nccl.CommDestroy = (int (*)(void*))dlsym(h, "ncclCommDestroy");
    g_nccl.GetErrorString = (const char* (*)(int))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllGather || !g_nccl.CommDestroy) {
        dlclose(h);
        return fail(BMTK_E_COMM, "'%s' lacks the NCCL entry points", p);
    }
    g_nccl.handle = h;
    return BMTK_OK;
}
constexpr int kNcclUint32 = 3;  // ncclUint32 in nccl.h's ncclDataType_t

}  // namespace bmtk

using namespace bmtk;

struct bmtk_engine {
    int device = 0;
    double dt = 0.1;
    cudaStream_t stream = nullptr;
    bool finalized = false;

    // nodes
    uint64_t n_global = 0, lo = 0, n_local = 0, n_virtual = 0;
    uint32_t n_pad = 0, n_pad1 = 0, n_trials = 1, trial_base = 0;
    std::vector<uint16_t> type_index;
    std::vector<bmtk_glif_params> types;
    bool has_theta = false;

    // edges (host accumulators until finalize)
    std::vector<uint32_t> e_src, e_trg;
    std::vector<float> e_w;
    std::vector<uint16_t> e_delay;
    std::vector<uint8_t> e_port;
    uint64_t n_edges = 0;
    uint32_t max_delay = 1, min_delay = 0, target_bits = 1, ring_slots = 2;

    // options
    bool deterministic = false, use_graph = true, record_spikes = false, profile = false;
    uint32_t window_opt = 0, window = 1;
    uint64_t spike_cap_opt = 0, log_cap = 1u << 23, event_cap = 1u << 22, chunk_steps = 4096;
    uint32_t send_cap = 0, virt_cap = 0;

    // comm
    void* comm = nullptr;
    int rank = 0, n_ranks = 1;

    // device memory
    StateSoA st{};
    uint16_t* d_type = nullptr;
    TypeConsts* d_types = nullptr;
    float* ring = nullptr;
    Ctl* d_ctl = nullptr;
    unsigned long long* d_rowptr = nullptr;
    uint2* d_entries = nullptr;
    uint32_t *d_send = nullptr, *d_gathered = nullptr, *d_virt = nullptr;
    uint32_t *d_log_stamp = nullptr, *d_log_id = nullptr;
    uint4* d_poisson_thr = nullptr;
    uint64_t seed = 0;
    std::vector<float> poisson_rates;
    bool has_poisson = false;

    // replayed input spikes
    uint32_t *d_in_ptr = nullptr, *d_in_step = nullptr, *d_in_src = nullptr;
    uint64_t in_ptr_base = 0;
    uint32_t in_ptr_len = 0;
    std::vector<uint32_t> pending_in_virt, pending_in_stamp, h_in_ptr, h_in_step, h_in_src;
    size_t in_cap = 0, in_ptr_cap = 0;
    bool has_pending_inputs = false;

    // clamps
    std::vector<uint64_t> ce_step;
    uint32_t* d_ce_target = nullptr;
    float* d_ce_delta = nullptr;
    size_t ce_next = 0;
    bool has_iext = false;
    std::vector<uint64_t> ce_step_in;
    std::vector<uint32_t> ce_target_in;
    std::vector<float> ce_delta_in;

    // probes
    std::vector<uint32_t> probe_ids;
    uint32_t probe_interval = 1;
    uint32_t n_probe_vars = 1, probe_vars = BMTK_VAR_V_M;   // recorded variables, 4 bits per code
    uint32_t* d_probe_ids = nullptr;
    float* d_trace = nullptr;
    uint32_t trace_cap = 0;
    uint64_t samples_drained = 0;
    std::vector<float> h_trace;

    // host store of recorded spikes: keys stamp << 32 | id, sorted (every drain appends a later, sorted run)
    // recorded spikes, (stamp, id)-sorted, in pinned host blocks of kSpkBlock entries ({stamps | ids});
    // blocks are added as the store grows and kept for re-use after a fetch (pinning memory is slow)
    static constexpr size_t kSpkBlock = 1u << 21;
    std::vector<uint32_t*> h_spk_blocks;
    size_t h_spk_n = 0;
    uint64_t log_base_step = 0;       // every stamp in the device log is greater than this
    unsigned long long *d_log_keys = nullptr, *d_log_keys2 = nullptr;
    void* d_log_tmp = nullptr;
    size_t log_tmp_bytes = 0;
    uint64_t step = 0;
    uint64_t launches = 0;
    uint64_t events_total = 0, spikes_total = 0, input_spikes_total = 0;

    // graph
    cudaGraphExec_t graph_exec = nullptr;
    bool graph_valid = false;

    // profiling
    std::vector<cudaEvent_t> ev_pool;
    std::vector<std::pair<int, int>> ev_update, ev_prop;  // indices into ev_pool
    double update_ns = 0, prop_ns = 0;
    uint64_t update_launches = 0, prop_launches = 0;

    // persistent stepping (single rank, atomic delivery)
    bool persistent = true, phase_timers = false, ring_prefetch = false;
    uint32_t tune = 0;
    // Overflow of a fixed-capacity list inside a chunk: the chunk is replayed from a device-side copy of the state it
    // started from, with the list that overflowed doubled (one rank; with several ranks capacities are part of the
    // agreed exchange layout and the error is returned).
    bool replay = true;
    std::vector<void*> bk_arrays;      // copies of ckpt_arrays(), in that order
    Ctl* d_bk_ctl = nullptr;
    uint32_t last_overflow = 0;        // device flags of the last overflow drain() saw
    uint64_t replays = 0;
    bool pipe_demoted = false;         // this chunk is replayed with the two-phase kernel
    uint32_t pipe_blocks_opt = 0;   // option pipeline_blocks: fewer blocks than SMs (a small network needs few update warps,
                                    // and a hand-over over fewer blocks is cheaper)
    int persist_blocks = 0;
    bool persist_resident = false;
    uint4* d_pipe_seg = nullptr;
    uint32_t pipe_warps_opt = 0;         // option pipeline_warps: 0 = choose, else 12 or 20 warps per block
    bool ring_stage = true;              // pipelined kernel: next step's ring cells copied to shared memory ahead (option ring_stage)
    uint32_t pipe_trials = 1, pipe_trials_opt = 0;   // trials one launch of the pipelined kernel steps (option pipeline_trials)
    uint32_t* d_pipe_sync = nullptr;     // pipelined kernel: the two phase counters
    uint32_t* d_log_seg_cnt = nullptr;   // pipelined kernel: spikes each block logged in the last launch
    unsigned long long* d_blk_prof = nullptr;   // pipelined kernel: per-block busy / wait sums (option phase_timers)
    bool log_segmented = false;          // the device log of the current chunk is in per-block segments
    bool pipeline = true;     // option: use the pipelined kernel where it applies
    bool pipe_ok = false;     // resident state, one trial, min delay >= 2 steps
    int pipe_blocks = 0;
    uint32_t pipe_upd_warps = 0;   // update warps per block: what the network needs at 128 neurons per warp
    uint32_t* d_virt2 = nullptr;
    uint4* d_plists[2] = {nullptr, nullptr};
    uint32_t* d_plist_counts = nullptr;
    // spike exchange over peer memory (several ranks, persistent kernel)
    unsigned long long* d_xchg = nullptr;             // this rank's exchange buffer
    unsigned long long* xchg_peers[kXRanks] = {};     // every rank's buffer as mapped here
    bool p2p_ready = false, p2p_by_pointer = false;
    // Exchange layout agreed between the ranks. set_global_layout supplies the network-wide minimum delay,
    // the largest block and whether any rank has clamp changes; window, spike capacity and the offsets
    // inside an exchange buffer follow from those, so every rank computes the same numbers. The first
    // kXDescWords words of an exchange buffer describe the layout its owner uses; p2p_connect compares.
    bool g_layout_set = false, g_any_clamps = false;
    uint64_t g_min_delay = 0, g_max_local = 0;
    bool peers_pipe_ok = true;   // every rank can run the pipelined kernel
    bool any_iext = false;       // some rank has clamp changes (the pipelined exchange has no clamp schedule)
    uint32_t xchg_seq = 0;                      // windows exchanged so far
    uint32_t pingpong_calls = 0;
    uint32_t xp_off = 0;                        // pipelined kernel: start of its exchange area (64-bit words)
    int32_t* d_probe_slot = nullptr;
    unsigned long long* d_ce_group_step = nullptr;
    uint32_t* d_ce_group_ptr = nullptr;
    std::vector<uint64_t> ce_group_step;
    size_t ce_group_next = 0;
    double phase_update_ns = 0, phase_prop_ns = 0, phase_sync1_ns = 0, phase_sync2_ns = 0;
    double phase_rows_ns = 0, phase_remote_wait_ns = 0, phase_remote_rows_ns = 0;
    double drain_wait_ns = 0, drain_sort_ns = 0;   // host clock: waiting for the chunk's kernels; sorting + copying its spike log
    uint64_t phase_windows = 0;

    DetWorkspace det{};
    cudaEvent_t marks[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

namespace bmtk {

constexpr uint32_t kXDescWords = 16;
constexpr unsigned long long kXDescMagic = 0x424d544b58444553ull;   // "BMTKXDES"

// What a rank's exchange buffer is laid out for (see bmtk_engine_exchange_layout in the header).
static void describe_layout(const bmtk_engine* e, uint64_t* d) {
    std::memset(d, 0, 8 * kXDescWords);
    d[0] = kXDescMagic;
    d[1] = (uint64_t)e->n_ranks;
    d[2] = e->window;
    d[3] = e->send_cap;
    d[4] = e->xp_off;
    d[5] = (uint64_t)e->persist_blocks;
    d[6] = (uint64_t)e->pipe_blocks;
    d[7] = (e->pipeline && e->pipe_ok) ? 1 : 0;
    d[8] = e->has_iext ? 1 : 0;
    d[9] = e->n_global;
    d[10] = e->n_virtual;
    std::memcpy(&d[11], &e->dt, 8);
    d[12] = e->max_delay;
}

// Two ranks can exchange spikes only if these agree; words 7 and 8 may differ (they are combined).
static int compare_layout(const uint64_t* a, const uint64_t* b, int rank_b) {
    static const char* names[kXDescWords] = {"magic", "number of ranks", "exchange window (steps)", "spike capacity",
                                             "offset of the pipelined exchange area", "blocks of the two-phase kernel",
                                             "blocks of the pipelined kernel", "", "", "number of neurons",
                                             "number of virtual cells", "dt", "", "", "", ""};
    for (uint32_t i = 0; i < kXDescWords; ++i) {
        if (!names[i][0] || a[i] == b[i]) continue;
        return fail(BMTK_E_INVALID, "exchange layout differs from rank %d: %s is %llu here and %llu there; give every rank "
                    "the same network-wide values with bmtk_engine_set_global_layout before finalize", rank_b, names[i],
                    (unsigned long long)a[i], (unsigned long long)b[i]);
    }
    return BMTK_OK;
}

static int set_device(bmtk_engine* e) {
    CU(cudaSetDevice(e->device));
    return BMTK_OK;
}

static IdSpace make_ids(bmtk_engine* e) {
    IdSpace s{};
    s.n_virtual = e->n_virtual ? (uint32_t)e->n_virtual : 1u;
    s.n_global = (uint32_t)e->n_global;
    if (e->n_trials > 1) {
        s.n_pad1 = e->n_pad1;
        s.n_cells_all = e->n_pad;
    } else {
        s.n_pad1 = (uint32_t)std::max<uint64_t>(e->n_global, 1);
        s.n_cells_all = (uint32_t)e->n_global;
    }
    return s;
}

static UpdateArgs make_update_args(bmtk_engine* e, uint32_t s) {
    UpdateArgs a{};
    a.st = e->st;
    a.types = e->d_types;
    a.n_types = (int32_t)e->types.size();
    a.n_local = (uint32_t)e->n_local;
    a.n_pad = e->n_pad;
    a.n_pad1 = e->n_pad1;
    a.ids = make_ids(e);
    a.n_trials = e->n_trials;
    a.trial_base = e->trial_base;
    a.lo = (uint32_t)e->lo;
    a.ring = e->ring;
    a.ring_slots = e->ring_slots;
    a.ctl = e->d_ctl;
    a.step_in_window = s;
    a.send = e->d_send;
    a.send_cap = e->send_cap;
    a.log_stamp = e->record_spikes ? e->d_log_stamp : nullptr;
    a.log_id = e->d_log_id;
    a.log_cap = (uint32_t)e->log_cap;
    a.poisson_thr = e->has_poisson ? e->d_poisson_thr : nullptr;
    a.n_virtual = (uint32_t)e->n_virtual;
    a.n_global = (uint32_t)e->n_global;
    a.seed = e->seed;
    a.virt = e->d_virt;
    a.virt_cap = e->virt_cap;
    return a;
}

static PropArgs make_prop_args(bmtk_engine* e, uint32_t w) {
    PropArgs a{};
    a.rowptr = e->d_rowptr;
    a.entries = e->d_entries;
    a.target_bits = e->target_bits;
    a.ring = e->ring;
    a.ring_slots = e->ring_slots;
    a.n_pad = e->n_pad;
    a.n_pad1 = e->n_pad1;
    a.ids = make_ids(e);
    a.ctl = e->d_ctl;
    a.gathered = e->n_ranks > 1 ? e->d_gathered : e->d_send;
    a.n_seg = (uint32_t)e->n_ranks;
    a.seg_stride = e->send_cap + 4;
    a.seg_cap = e->send_cap;
    a.in_ptr = e->d_in_ptr;
    a.in_ptr_base = e->in_ptr_base;
    a.in_ptr_len = e->in_ptr_len;
    a.in_step = e->d_in_step;
    a.in_src = e->d_in_src;
    a.virt = e->has_poisson ? e->d_virt : nullptr;
    a.virt_cap = e->virt_cap;
    a.window = w;
    a.send = e->d_send;
    return a;
}

static int get_event(bmtk_engine* e, int* idx) {
    cudaEvent_t ev;
    CU(cudaEventCreate(&ev));
    e->ev_pool.push_back(ev);
    *idx = (int)e->ev_pool.size() - 1;
    return BMTK_OK;
}

// Enqueues one window of `w` steps starting at host step e->step. `capturing` skips everything
// that cannot be part of a graph (profiling events, clamp launches).
static int enqueue_window(bmtk_engine* e, uint32_t w, bool capturing) {
    for (uint32_t s = 0; s < w; ++s) {
        if (!capturing && e->has_iext) {
            const uint64_t n = e->step + s;
            size_t b = e->ce_next;
            while (e->ce_next < e->ce_step.size() && e->ce_step[e->ce_next] <= n) ++e->ce_next;
            if (e->ce_next > b) {
                const uint32_t cnt = (uint32_t)(e->ce_next - b);
                apply_clamp_kernel<<<(cnt + 127) / 128, 128, 0, e->stream>>>(e->st.i_ext, e->d_ce_target, e->d_ce_delta,
                                                                            (uint32_t)b, (uint32_t)e->ce_next,
                                                                            (uint32_t)e->lo);
                CU(cudaGetLastError());
                ++e->launches;
            }
        }
        int e0 = -1, e1 = -1;
        if (e->profile && !capturing) {
            int rc = get_event(e, &e0);
            if (rc) return rc;
            CU(cudaEventRecord(e->ev_pool[e0], e->stream));
        }
        const UpdateArgs ua = make_update_args(e, s);
        CU(launch_glif_update(ua, e->has_theta, e->has_iext, e->stream));
        ++e->launches;
        if (e->profile && !capturing) {
            int rc = get_event(e, &e1);
            if (rc) return rc;
            CU(cudaEventRecord(e->ev_pool[e1], e->stream));
            e->ev_update.emplace_back(e0, e1);
        }
        if (!e->probe_ids.empty()) {
            const uint32_t n_ids = (uint32_t)e->probe_ids.size();
            const int blocks = (int)std::min<uint32_t>((n_ids + 255) / 256, 148 * 4);
            snapshot_kernel<<<blocks, 256, 0, e->stream>>>(e->d_ctl, s, e->probe_interval, e->d_probe_ids, n_ids, e->st, e->n_pad,
                                                           e->d_types, e->d_trace, e->trace_cap, e->n_probe_vars, e->probe_vars);
            CU(cudaGetLastError());
            ++e->launches;
        }
    }
    if (e->n_ranks > 1) {
        if (!e->comm) return fail(BMTK_E_COMM, "several ranks without an NCCL communicator: connect the peer-memory exchange "
                                  "(p2p_connect) or pass an id to comm_init");
        const int rc = g_nccl.AllGather(e->d_send, e->d_gathered, (size_t)e->send_cap + 4, kNcclUint32, e->comm,
                                        e->stream);
        if (rc != 0)
            return fail(BMTK_E_COMM, "ncclAllGather failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
    }
    const PropArgs pa = make_prop_args(e, w);
    int p0 = -1, p1 = -1;
    if (e->profile && !capturing) {
        int rc = get_event(e, &p0);
        if (rc) return rc;
        CU(cudaEventRecord(e->ev_pool[p0], e->stream));
    }
    if (e->deterministic) {
        const int rc = propagate_det_window(pa, e->det, e->stream, &e->launches);
        if (rc == -2) return fail(BMTK_E_OVERFLOW, "deterministic propagate: more than %llu events in one window "
                                  "(raise option event_capacity)", (unsigned long long)e->event_cap);
        if (rc != 0) return fail(BMTK_E_CUDA, "deterministic propagate failed: %s", cudaGetErrorString(cudaGetLastError()));
    } else {
        CU(launch_propagate_atomic(pa, e->stream));
        ++e->launches;
    }
    if (e->profile && !capturing) {
        int rc = get_event(e, &p1);
        if (rc) return rc;
        CU(cudaEventRecord(e->ev_pool[p1], e->stream));
        e->ev_prop.emplace_back(p0, p1);
    }
    return BMTK_OK;
}

static void drop_graph(bmtk_engine* e) {
    if (e->graph_exec) cudaGraphExecDestroy(e->graph_exec);
    e->graph_exec = nullptr;
    e->graph_valid = false;
}

static int capture_graph(bmtk_engine* e) {
    drop_graph(e);
    cudaGraph_t graph = nullptr;
    CU(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const uint64_t launches_before = e->launches;
    const int rc = enqueue_window(e, e->window, true);
    e->launches = launches_before;
    cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
    if (rc != BMTK_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
    ce = cudaGraphInstantiate(&e->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "graph instantiate failed: %s", cudaGetErrorString(ce));
    e->graph_valid = true;
    return BMTK_OK;
}

static uint32_t launches_per_window(bmtk_engine* e, uint32_t w) {
    return w * (1u + (e->probe_ids.empty() ? 0u : 1u)) + 1u;
}

// Uploads pending replay spikes: keeps stamps > current step, sorts by emitting step, builds the
// per-step pointer table.
static int upload_inputs(bmtk_engine* e) {
    if (!e->has_pending_inputs) return BMTK_OK;
    e->has_pending_inputs = false;
    drop_graph(e);
    const size_t n_in = e->pending_in_virt.size();
    // keep stamps > current step; counting sort by emitting step (= stamp - 1) gives the pointer table
    const uint64_t base = e->step;
    uint64_t last = 0;
    size_t n_keep = 0;
    for (size_t i = 0; i < n_in; ++i) {
        const uint64_t stamp = e->pending_in_stamp[i];
        if (stamp <= base) continue;
        ++n_keep;
        if (stamp - 1 > last) last = stamp - 1;
    }
    e->in_ptr_len = 0;
    if (n_keep == 0) {
        e->pending_in_virt.clear();
        e->pending_in_stamp.clear();
        cudaFree(e->d_in_ptr); cudaFree(e->d_in_step); cudaFree(e->d_in_src);
        e->d_in_ptr = e->d_in_step = e->d_in_src = nullptr;
        e->in_cap = e->in_ptr_cap = 0;
        return BMTK_OK;
    }
    const uint64_t len = last - base + 2;  // entries for steps base..last, plus the end
    if (len > (1ull << 31)) return fail(BMTK_E_INVALID, "input spikes span too many steps");
    std::vector<uint32_t>& ptr = e->h_in_ptr;
    ptr.assign(len, 0u);
    for (size_t i = 0; i < n_in; ++i) {
        const uint64_t stamp = e->pending_in_stamp[i];
        if (stamp > base) ++ptr[stamp - 1 - base + 1];
    }
    for (uint64_t i = 1; i < len; ++i) ptr[i] += ptr[i - 1];
    std::vector<uint32_t>& st = e->h_in_step;
    std::vector<uint32_t>& sr = e->h_in_src;
    st.resize(n_keep);
    sr.resize(n_keep);
    std::vector<uint32_t> fill(ptr.begin(), ptr.end() - 1);
    for (size_t i = 0; i < n_in; ++i) {
        const uint64_t stamp = e->pending_in_stamp[i];
        if (stamp <= base) continue;
        const uint32_t pos = fill[stamp - 1 - base]++;
        st[pos] = (uint32_t)(stamp - 1);
        sr[pos] = (uint32_t)(e->n_global + e->pending_in_virt[i]);
    }
    e->pending_in_virt.clear();
    e->pending_in_stamp.clear();
    if (len > e->in_ptr_cap) {
        cudaFree(e->d_in_ptr);
        e->d_in_ptr = nullptr;
        e->in_ptr_cap = len + len / 2;
        CU(cudaMalloc(&e->d_in_ptr, 4 * e->in_ptr_cap));
    }
    if (n_keep > e->in_cap) {
        cudaFree(e->d_in_step); cudaFree(e->d_in_src);
        e->d_in_step = e->d_in_src = nullptr;
        e->in_cap = n_keep + n_keep / 2;
        CU(cudaMalloc(&e->d_in_step, 4 * e->in_cap));
        CU(cudaMalloc(&e->d_in_src, 4 * e->in_cap));
    }
    CU(cudaMemcpyAsync(e->d_in_ptr, ptr.data(), 4 * len, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_in_step, st.data(), 4 * n_keep, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_in_src, sr.data(), 4 * n_keep, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    e->in_ptr_base = base;
    e->in_ptr_len = (uint32_t)len;
    return BMTK_OK;
}

// The dynamic state of an engine: neuron state arrays and the ring buffer (what a checkpoint holds and what a
// replayed chunk starts from again).
struct CkptArray {
    void* dev;
    size_t bytes;
};
std::vector<CkptArray> ckpt_arrays(bmtk_engine* e) {
    const size_t np = e->n_pad;
    std::vector<CkptArray> v = {
        {e->st.U, 4 * np}, {e->st.asc0, 4 * np}, {e->st.asc1, 4 * np}, {e->st.y1, 4 * np * kPorts},
        {e->st.y2, 4 * np * kPorts}, {e->st.refr, 4 * np}, {e->ring, 4 * (size_t)e->ring_slots * kPorts * np}};
    if (e->has_theta) {
        v.push_back({e->st.th_spike, 4 * np});
        v.push_back({e->st.th_voltage, 4 * np});
    }
    if (e->has_iext) v.push_back({e->st.i_ext, 4 * np});
    return v;
}

// Copies the dynamic state and the control block aside (device to device) before a chunk runs.
static int backup_state(bmtk_engine* e) {
    const std::vector<CkptArray> arrs = ckpt_arrays(e);
    if (e->bk_arrays.empty()) {
        for (const CkptArray& a : arrs) {
            void* p = nullptr;
            CU(cudaMalloc(&p, a.bytes));
            e->bk_arrays.push_back(p);
        }
        CU(cudaMalloc(&e->d_bk_ctl, sizeof(Ctl)));
    }
    for (size_t i = 0; i < arrs.size(); ++i)
        CU(cudaMemcpyAsync(e->bk_arrays[i], arrs[i].dev, arrs[i].bytes, cudaMemcpyDeviceToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_bk_ctl, e->d_ctl, sizeof(Ctl), cudaMemcpyDeviceToDevice, e->stream));
    return BMTK_OK;
}

static int realloc_dev(void** p, size_t bytes) {
    cudaFree(*p);
    *p = nullptr;
    CU(cudaMalloc(p, bytes));
    return BMTK_OK;
}

// After an overflow: the state the chunk started from comes back, the lists are emptied, the host clock is set
// back by `chunk` steps, and whatever overflowed (device flags `f`, or the deterministic delivery's event list when
// f == 0) is doubled.
static int restore_and_grow(bmtk_engine* e, uint64_t chunk_start, uint32_t f) {
    CU(cudaStreamSynchronize(e->stream));
    const std::vector<CkptArray> arrs = ckpt_arrays(e);
    for (size_t i = 0; i < arrs.size(); ++i)
        CU(cudaMemcpyAsync(arrs[i].dev, e->bk_arrays[i], arrs[i].bytes, cudaMemcpyDeviceToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_ctl, e->d_bk_ctl, sizeof(Ctl), cudaMemcpyDeviceToDevice, e->stream));
    e->step = chunk_start;
    e->ce_next = 0;
    while (e->ce_next < e->ce_step.size() && e->ce_step[e->ce_next] < e->step) ++e->ce_next;
    e->ce_group_next = 0;
    while (e->ce_group_next < e->ce_group_step.size() && e->ce_group_step[e->ce_group_next] < e->step) ++e->ce_group_next;
    e->log_segmented = false;
    drop_graph(e);
    int rc = BMTK_OK;
    if (f & kErrLogFull) {
        if (e->log_cap * 2 >= (1ull << 32)) return fail(BMTK_E_OVERFLOW, "spike log cannot grow beyond 2^32 entries");
        e->log_cap *= 2;
        if ((rc = realloc_dev((void**)&e->d_log_stamp, 4 * e->log_cap))) return rc;
        if ((rc = realloc_dev((void**)&e->d_log_id, 4 * e->log_cap))) return rc;
        if ((rc = realloc_dev((void**)&e->d_log_keys, 8 * e->log_cap))) return rc;
        if ((rc = realloc_dev((void**)&e->d_log_keys2, 8 * e->log_cap))) return rc;
        e->log_tmp_bytes = spike_log_sort_tmp_bytes((uint32_t)e->log_cap);
        if ((rc = realloc_dev(&e->d_log_tmp, e->log_tmp_bytes))) return rc;
    }
    if (f & kErrSpikeListFull) {
        // the pipelined kernel's lists are per block and fixed: this chunk runs on the two-phase kernel, whose
        // window list can grow
        e->pipe_demoted = true;
        if ((uint64_t)e->send_cap * 2 + 4 >= (1ull << 31)) return fail(BMTK_E_OVERFLOW, "spike list cannot grow further");
        e->send_cap *= 2;
        const size_t seg = (size_t)e->send_cap + 4;
        if ((rc = realloc_dev((void**)&e->d_send, 4 * seg))) return rc;
        for (int q = 0; q < 2; ++q)
            if (e->d_plists[q] && (rc = realloc_dev((void**)&e->d_plists[q], sizeof(uint4) * (size_t)e->send_cap))) return rc;
    }
    if (f & kErrVirtListFull) {
        e->virt_cap *= 2;
        if ((rc = realloc_dev((void**)&e->d_virt, 4 * ((size_t)e->virt_cap + 4)))) return rc;
        if (e->d_virt2 && (rc = realloc_dev((void**)&e->d_virt2, 4 * ((size_t)e->virt_cap + 4)))) return rc;
    }
    if (e->deterministic && (f == 0 || (f & (kErrSpikeListFull | kErrVirtListFull | kErrEventsFull)))) {
        if (f == 0 || (f & kErrEventsFull)) e->event_cap *= 2;
        if (e->event_cap >= (1ull << 31)) return fail(BMTK_E_OVERFLOW, "event list cannot grow beyond 2^31 entries");
        det_free(e->det);
        const uint64_t ring_cells = (uint64_t)e->ring_slots * kPorts * e->n_pad;
        if (det_alloc(e->det, (uint32_t)e->event_cap, (uint32_t)((size_t)e->send_cap * e->n_ranks + e->virt_cap + 65536),
                      ring_cells) != cudaSuccess)
            return fail(BMTK_E_CUDA, "deterministic workspace could not grow");
    }
    // empty lists, and no descriptor of the failed attempt may be taken for one of the replay (same tags)
    CU(cudaMemsetAsync(e->d_send, 0, 4 * ((size_t)e->send_cap + 4), e->stream));
    if (e->d_virt) CU(cudaMemsetAsync(e->d_virt, 0, 4, e->stream));
    if (e->d_virt2) CU(cudaMemsetAsync(e->d_virt2, 0, 4, e->stream));
    if (e->d_plist_counts) CU(cudaMemsetAsync(e->d_plist_counts, 0, 8, e->stream));
    if (e->d_pipe_seg) CU(cudaMemsetAsync(e->d_pipe_seg, 0, sizeof(uint4) * 3 * (size_t)e->pipe_blocks * kPipeSegCap, e->stream));
    if (e->d_log_seg_cnt) CU(cudaMemsetAsync(e->d_log_seg_cnt, 0, 4 * (size_t)e->pipe_blocks, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    ++e->replays;
    return BMTK_OK;
}

// Brings counters, spike log and traces of the finished chunk to the host.
static double now_ns() {
    return (double)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch()).count();
}

static int drain(bmtk_engine* e) {
    Ctl h{};
    const double t0 = now_ns();
    CU(cudaMemcpyAsync(&h, e->d_ctl, sizeof(Ctl), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    const double t1 = now_ns();
    e->drain_wait_ns += t1 - t0;
    e->events_total = h.n_events;
    e->spikes_total = h.n_spikes;
    e->input_spikes_total = h.n_input_spikes;
    if (h.n_windows) {
        e->phase_update_ns += (double)h.t_update_ns;
        e->phase_prop_ns += (double)h.t_prop_ns;
        e->phase_windows += h.n_windows;
        e->phase_sync1_ns += (double)h.t_sync1_ns;
        e->phase_sync2_ns += (double)h.t_sync2_ns;
        e->phase_rows_ns += (double)h.t_rows_ns;
        e->phase_remote_wait_ns += (double)h.t_remote_wait_ns;
        e->phase_remote_rows_ns += (double)h.t_remote_rows_ns;
        CU(cudaMemsetAsync(&e->d_ctl->t_update_ns, 0, sizeof(Ctl) - offsetof(Ctl, t_update_ns), e->stream));
    }
    if (h.step_base != e->step)
        return fail(BMTK_E_INVALID, "device clock %llu differs from host clock %llu", (unsigned long long)h.step_base,
                    (unsigned long long)e->step);
    if (e->profile) {
        for (auto& pr : e->ev_update) {
            float ms = 0;
            CU(cudaEventElapsedTime(&ms, e->ev_pool[pr.first], e->ev_pool[pr.second]));
            e->update_ns += (double)ms * 1e6;
            ++e->update_launches;
        }
        for (auto& pr : e->ev_prop) {
            float ms = 0;
            CU(cudaEventElapsedTime(&ms, e->ev_pool[pr.first], e->ev_pool[pr.second]));
            e->prop_ns += (double)ms * 1e6;
            ++e->prop_launches;
        }
        for (auto ev : e->ev_pool) cudaEventDestroy(ev);
        e->ev_pool.clear();
        e->ev_update.clear();
        e->ev_prop.clear();
    }
    if (h.error_flags) {
        const uint32_t f = h.error_flags;
        e->last_overflow = f;
        CU(cudaMemsetAsync(&e->d_ctl->error_flags, 0, 4, e->stream));
        if (f & kErrSpikeListFull)
            return fail(BMTK_E_OVERFLOW, "window spike list full (capacity %u per rank; the persistent kernel also holds "
                        "at most 4096 spikes per block and window, the pipelined kernel 2048 per block and phase): raise option "
                        "spike_capacity, or set pipeline = 0 or persistent = 0",
                        e->send_cap);
        if (f & kErrExchangeTimeout)
            return fail(BMTK_E_COMM, "spike exchange timed out: a rank did not publish its window within ~1 s "
                        "(rank %d of %d); the results of this run are invalid", e->rank, e->n_ranks);
        if (f & kErrBadChunk)
            return fail(BMTK_E_CUDA, "pipelined kernel: a chunk descriptor outside the CSR was read (a list was not complete); "
                        "the results of this run are invalid (set option pipeline = 0)");
        if (f & kErrSyncTimeout)
            return fail(BMTK_E_CUDA, "pipelined kernel: a phase hand-over between update and delivery warps timed out; "
                        "the results of this run are invalid (set option pipeline = 0)");
        if (f & kErrVirtListFull)
            return fail(BMTK_E_OVERFLOW, "Poisson spike list full (capacity %u): raise option spike_capacity", e->virt_cap);
        if (f & kErrLogFull)
            return fail(BMTK_E_OVERFLOW, "spike log full (capacity %llu, split evenly over the blocks of the pipelined kernel): raise log_capacity or lower chunk_steps",
                        (unsigned long long)e->log_cap);
        return fail(BMTK_E_OVERFLOW, "device buffer overflow (flags %u)", f);
    }
    if (e->record_spikes && h.log_count) {
        // sort the chunk's spikes by (stamp, id) on the device; chunks are consecutive in time, so the
        // host store stays sorted by appending
        const size_t n0 = e->h_spk_n, n = h.log_count;
        auto bits_for = [](uint64_t v) { uint32_t b = 1; while (b < 64 && (v >> b)) ++b; return b; };
        const uint32_t stamp_bits = bits_for(e->step - e->log_base_step + 1);
        const uint32_t id_bits = bits_for(std::max<uint64_t>(e->n_global, e->n_pad));
        CU(sort_spike_log((uint32_t)n, e->d_log_stamp, e->d_log_id, (uint32_t)e->log_base_step, stamp_bits, id_bits,
                          e->d_log_keys, e->d_log_keys2, e->d_log_tmp, e->log_tmp_bytes, e->stream,
                          e->log_segmented ? (uint32_t)e->pipe_blocks : 0u, (uint32_t)(e->log_cap / std::max(e->pipe_blocks, 1)),
                          e->d_log_seg_cnt));
        e->launches += 3;
        // straight into the host store: chunks are consecutive in time, so it stays (stamp, id)-sorted
        constexpr size_t B = bmtk_engine::kSpkBlock;
        for (size_t done = 0; done < n;) {
            const size_t pos = n0 + done, blk = pos / B, off = pos % B, take = std::min(n - done, B - off);
            if (blk == e->h_spk_blocks.size()) {
                uint32_t* p = nullptr;
                CU(cudaMallocHost(&p, 4 * 2 * B));
                e->h_spk_blocks.push_back(p);
            }
            uint32_t* p = e->h_spk_blocks[blk];
            CU(cudaMemcpyAsync(p + off, e->d_log_stamp + done, 4 * take, cudaMemcpyDeviceToHost, e->stream));
            CU(cudaMemcpyAsync(p + B + off, e->d_log_id + done, 4 * take, cudaMemcpyDeviceToHost, e->stream));
            done += take;
        }
        CU(cudaMemsetAsync(&e->d_ctl->log_count, 0, 4, e->stream));
        CU(cudaStreamSynchronize(e->stream));
        e->h_spk_n = n0 + n;
        e->drain_sort_ns += now_ns() - t1;
    }
    e->log_base_step = e->step;
    e->log_segmented = false;
    if (!e->probe_ids.empty()) {
        const uint64_t have = e->step / e->probe_interval;
        const uint64_t n_new = have - e->samples_drained;
        if (n_new) {
            const size_t n_ids = e->probe_ids.size() * e->n_probe_vars, n0 = e->h_trace.size();   // values per sample
            e->h_trace.resize(n0 + n_new * n_ids);
            CU(cudaMemcpyAsync(e->h_trace.data() + n0, e->d_trace, 4 * n_new * n_ids, cudaMemcpyDeviceToHost, e->stream));
            e->samples_drained = have;
            const uint32_t sb = (uint32_t)have;
            CU(cudaMemcpyAsync(&e->d_ctl->sample_base, &sb, 4, cudaMemcpyHostToDevice, e->stream));
            CU(cudaStreamSynchronize(e->stream));
        }
    }
    return BMTK_OK;
}

// The pipelined kernel runs when this rank can (resident state, min delay >= 2 steps) and,
// with several ranks, when every rank can and none has clamp changes: the ranks must all run the same
// exchange protocol.
static bool use_pipelined(const bmtk_engine* e) {
    if (!e->pipeline || !e->pipe_ok || e->pipe_demoted) return false;
    if (e->n_ranks == 1) return true;
    return e->p2p_ready && e->peers_pipe_ok && !e->any_iext;
}

// One cooperative launch that executes `n` steps (update + delivery of every window inside it).
static int run_persistent_chunk(bmtk_engine* e, uint32_t n) {
    PersistArgs a{};
    a.st = e->st;
    a.types = e->d_types;
    a.n_types = (int32_t)e->types.size();
    a.n_local = (uint32_t)e->n_local;
    a.n_pad = e->n_pad;
    a.lo = (uint32_t)e->lo;
    a.n_global = (uint32_t)e->n_global;
    a.n_pad1 = e->n_pad1;
    a.n_trials = e->n_trials;
    a.trial_base = e->trial_base;
    a.ids = make_ids(e);
    a.ring = e->ring;
    a.ring_slots = e->ring_slots;
    a.ctl = e->d_ctl;
    a.lists[0] = e->d_plists[0];
    a.lists[1] = e->d_plists[1];
    a.list_counts = e->d_plist_counts;
    a.send_cap = e->send_cap;
    a.log_stamp = e->record_spikes ? e->d_log_stamp : nullptr;
    a.log_id = e->d_log_id;
    a.log_cap = (uint32_t)e->log_cap;
    CU(cudaMemsetAsync(e->d_plist_counts, 0, 8, e->stream));
    a.poisson_thr = e->has_poisson ? e->d_poisson_thr : nullptr;
    a.n_virtual = (uint32_t)e->n_virtual;
    a.seed = e->seed;
    a.virts[0] = e->d_virt;
    a.virts[1] = e->d_virt2;
    a.virt_cap = e->virt_cap;
    a.rowptr = e->d_rowptr;
    a.entries = e->d_entries;
    a.target_bits = e->target_bits;
    a.in_ptr = e->d_in_ptr;
    a.in_ptr_base = e->in_ptr_base;
    a.in_ptr_len = e->in_ptr_len;
    a.in_step = e->d_in_step;
    a.in_src = e->d_in_src;
    a.n_steps = n;
    a.window = e->window;
    a.ce_group_step = e->d_ce_group_step;
    a.ce_group_ptr = e->d_ce_group_ptr;
    a.ce_group_begin = (uint32_t)e->ce_group_next;
    a.ce_group_end = (uint32_t)e->ce_group_step.size();
    a.ce_target = e->d_ce_target;
    a.ce_delta = e->d_ce_delta;
    a.probe_slot = e->probe_ids.empty() ? nullptr : e->d_probe_slot;
    a.n_probe = (uint32_t)e->probe_ids.size();
    a.probe_interval = e->probe_interval;
    a.n_probe_vars = e->n_probe_vars;
    a.probe_vars = e->probe_vars;
    a.trace = e->d_trace;
    a.trace_cap = e->trace_cap;
    a.profile = e->phase_timers ? 1u : 0u;
    a.ring_prefetch = e->ring_prefetch ? 1u : 0u;
    a.tune = e->tune;
    a.n_ranks = (uint32_t)e->n_ranks;
    a.rank = (uint32_t)e->rank;
    a.xchg_cap = e->send_cap;
    a.seq0 = e->xchg_seq;
    for (int r = 0; r < e->n_ranks; ++r) a.peers[r] = e->xchg_peers[r];
    const bool pipelined = use_pipelined(e);
    if (pipelined) {
        a.xp_off = e->xp_off;
        a.half = std::min<uint32_t>(e->window / 2, (uint32_t)kMaxWindow);
        a.pipe_seg = e->d_pipe_seg;
        a.pipe_seg_cap = kPipeSegCap;
        a.n_entries = e->n_edges;
        a.pipe_sync = e->d_pipe_sync;
        CU(cudaMemsetAsync(e->d_pipe_sync, 0, 32, e->stream));
        a.log_seg_cap = (uint32_t)(e->log_cap / e->pipe_blocks);
        a.log_seg_cnt = e->d_log_seg_cnt;
        e->log_segmented = e->record_spikes;
        a.upd_warps = e->pipe_upd_warps;
        a.blk_prof = e->phase_timers ? e->d_blk_prof : nullptr;
        // several trials: the chunk of steps is run for `pipe_trials` trials at a time, so that the ring slots the
        // launch scatters into stay in L2; one trial: a single launch over all cells
        const uint32_t per_launch = e->n_trials > 1 ? e->pipe_trials : 1u;
        a.ring_stage = (e->ring_stage && a.half > 1) ? 1u : 0u;
        // input warps: one thread per 2 Poisson cells of the block's share, at most half of the non-update warps;
        // replayed spikes alone get one warp
        {
            uint32_t iw = 0;
            if (e->has_poisson) iw = (uint32_t)((e->n_virtual * per_launch / e->pipe_blocks + 63) / 64);
            // always at least one: the input warps also queue the block's own spikes and write the spike log
            iw = std::max(iw, 1u);
            // the small block (12 warps, no register spills in the update) where it leaves at least 5 chunk warps: with
            // fewer the delivering side became the slower one (measured on 50 000 neurons x 1, 2, 3 trials per launch)
            const uint32_t others = e->pipe_upd_warps + iw + (e->n_ranks > 1 ? 1u : 0u);
            const bool small = e->pipe_warps_opt ? e->pipe_warps_opt == pipelined_warps_small()
                                                 : others + 5u <= pipelined_warps_small();
            a.block_warps = small && others + 1u <= pipelined_warps_small() ? pipelined_warps_small() : pipelined_warps();
            const uint32_t free_warps = a.block_warps - e->pipe_upd_warps;
            a.input_warps = std::max(1u, std::min(iw, free_warps / 2));
        }
        // the trials are dealt evenly to ceil(T / per_launch) launches (64 trials, 3 per launch: 20 x 3 + 2 x 2)
        const uint32_t n_launch = (e->n_trials + per_launch - 1) / per_launch;
        for (uint32_t g = 0, t0 = 0; g < n_launch; ++g) {
            const uint32_t nt = e->n_trials / n_launch + (g < e->n_trials % n_launch ? 1u : 0u);
            a.trial0 = t0;
            a.cell0 = t0 * e->n_pad1;
            a.n_cells = nt * e->n_pad1;
            a.log_append = g > 0;
            a.advance_clock = g + 1 == n_launch;
            t0 += nt;
            if (g > 0) {
                // the next trials run the same steps: counters start over, and no descriptor of the trials before
                // (valid by the tag of its phase) may be left where a neighbour looks for spill-over
                CU(cudaMemsetAsync(e->d_pipe_sync, 0, 32, e->stream));
                CU(cudaMemsetAsync(e->d_pipe_seg, 0, sizeof(uint4) * 3 * (size_t)e->pipe_blocks * kPipeSegCap, e->stream));
                ++e->launches;
            }
            CU(launch_pipelined(a, e->has_theta, e->has_iext, e->pipe_blocks, e->stream));
        }
    } else {
        CU(launch_persistent(a, e->has_theta, e->has_iext, e->persist_resident, e->persist_blocks, e->stream));
    }
    ++e->launches;
    e->step += n;
    // windows (two-phase kernel) or phases (pipelined kernel) exchanged so far: the same on every rank
    e->xchg_seq += pipelined ? (n + a.half - 1) / a.half : (n + e->window - 1) / e->window;
    // lists are empty at rest, whichever path runs next
    if (e->d_virt) CU(cudaMemsetAsync(e->d_virt, 0, 4, e->stream));
    if (e->d_virt2) CU(cudaMemsetAsync(e->d_virt2, 0, 4, e->stream));
    while (e->ce_group_next < e->ce_group_step.size() && e->ce_group_step[e->ce_group_next] < e->step) ++e->ce_group_next;
    while (e->ce_next < e->ce_step.size() && e->ce_step[e->ce_next] < e->step) ++e->ce_next;
    return BMTK_OK;
}

static int run_steps(bmtk_engine* e, uint64_t n_steps) {
    int rc = upload_inputs(e);
    if (rc) return rc;
    uint64_t left = n_steps;
    while (left) {
        uint64_t chunk = std::min<uint64_t>(left, e->chunk_steps);
        if (!e->probe_ids.empty()) {
            // the trace buffer holds trace_cap samples
            const uint64_t room = (uint64_t)e->trace_cap * e->probe_interval;
            chunk = std::min<uint64_t>(chunk, std::max<uint64_t>(room - e->probe_interval + 1, 1));
        }
        // one rank: keep what the chunk starts from, so that an overflow inside it can be answered by a replay
        const bool can_replay = e->replay && e->n_ranks == 1;
        const uint64_t chunk_start = e->step;
        if (can_replay) {
            rc = backup_state(e);
            if (rc) return rc;
        }
        int attempts = 0;
    again:
        uint64_t done = 0;
        const bool use_persistent = e->persistent && (e->n_ranks == 1 || e->p2p_ready) && !e->deterministic &&
                                    !e->profile && e->persist_blocks > 0;
        if (use_persistent) {
            rc = run_persistent_chunk(e, (uint32_t)chunk);
            if (rc) return rc;
            done = chunk;
        }
        while (done < chunk) {
            const uint32_t w = (uint32_t)std::min<uint64_t>(e->window, chunk - done);
            bool clamp_in_window = false;
            if (e->has_iext && e->ce_next < e->ce_step.size() && e->ce_step[e->ce_next] < e->step + w)
                clamp_in_window = true;
            const bool graph_ok = e->use_graph && !e->deterministic && !e->profile && w == e->window && !clamp_in_window;
            if (graph_ok) {
                if (!e->graph_valid) {
                    rc = capture_graph(e);
                    if (rc) return rc;
                }
                CU(cudaGraphLaunch(e->graph_exec, e->stream));
                e->launches += launches_per_window(e, w);
            } else {
                rc = enqueue_window(e, w, false);
                if (rc == BMTK_E_OVERFLOW && can_replay && attempts < 8) {
                    // the deterministic delivery found more events in a window than its lists hold
                    ++attempts;
                    e->last_overflow = 0;
                    rc = restore_and_grow(e, chunk_start, 0);
                    if (rc) return rc;
                    goto again;
                }
                if (rc) return rc;
            }
            e->step += w;
            done += w;
            while (e->ce_group_next < e->ce_group_step.size() && e->ce_group_step[e->ce_group_next] < e->step)
                ++e->ce_group_next;
        }
        rc = drain(e);
        if (rc == BMTK_E_OVERFLOW && can_replay && attempts < 8) {
            ++attempts;
            const std::string why = g_last_error;
            rc = restore_and_grow(e, chunk_start, e->last_overflow);
            if (rc) return rc;
            goto again;
        }
        e->pipe_demoted = false;
        if (rc) return rc;
        left -= chunk;
    }
    return BMTK_OK;
}

}  // namespace bmtk

// =============================================================================================
// C ABI

extern "C" {

const char* bmtk_last_error(void) { return g_last_error.c_str(); }
const char* bmtk_version(void) { return "bmtk_b200 0.1 sm_100a"; }

int bmtk_engine_create(bmtk_engine** out, int device, double dt_ms) {
    if (!out) return fail(BMTK_E_INVALID, "out is NULL");
    if (!(dt_ms > 0)) return fail(BMTK_E_INVALID, "dt must be positive");
    int n_dev = 0;
    cudaError_t ce = cudaGetDeviceCount(&n_dev);
    if (ce != cudaSuccess || n_dev == 0)
        return fail(BMTK_E_CUDA, "no CUDA device available (%s): this engine has no CPU path",
                    ce != cudaSuccess ? cudaGetErrorString(ce) : "device count 0");
    if (device < 0 || device >= n_dev) return fail(BMTK_E_INVALID, "device %d out of range (%d present)", device, n_dev);
    bmtk_engine* e = new bmtk_engine();
    e->device = device;
    e->dt = dt_ms;
    ce = cudaSetDevice(device);
    if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
    if (ce != cudaSuccess) {
        delete e;
        return fail(BMTK_E_CUDA, "cannot initialise device %d: %s", device, cudaGetErrorString(ce));
    }
    *out = e;
    return BMTK_OK;
}

int bmtk_engine_destroy(bmtk_engine* e) {
    if (!e) return BMTK_OK;
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    drop_graph(e);
    for (auto ev : e->ev_pool) cudaEventDestroy(ev);
    for (auto ev : e->marks) if (ev) cudaEventDestroy(ev);
    if (e->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(e->comm);
    det_free(e->det);
    cudaFree(e->st.U); cudaFree(e->st.asc0); cudaFree(e->st.asc1); cudaFree(e->st.y1); cudaFree(e->st.y2);
    cudaFree(e->st.refr); cudaFree(e->st.th_spike); cudaFree(e->st.th_voltage); cudaFree(e->st.i_ext);
    cudaFree(e->d_type); cudaFree(e->d_types); cudaFree(e->ring); cudaFree(e->d_ctl);
    cudaFree(e->d_rowptr); cudaFree(e->d_entries); cudaFree(e->d_send); cudaFree(e->d_gathered); cudaFree(e->d_virt);
    cudaFree(e->d_log_stamp); cudaFree(e->d_log_id); cudaFree(e->d_poisson_thr);
    cudaFree(e->d_in_ptr); cudaFree(e->d_in_step); cudaFree(e->d_in_src);
    cudaFree(e->d_ce_target); cudaFree(e->d_ce_delta); cudaFree(e->d_probe_ids); cudaFree(e->d_trace);
    cudaFree(e->d_virt2); cudaFree(e->d_probe_slot); cudaFree(e->d_ce_group_step); cudaFree(e->d_ce_group_ptr);
    cudaFree(e->d_plists[0]); cudaFree(e->d_plists[1]); cudaFree(e->d_plist_counts);
    for (int r = 0; r < e->n_ranks && r < (int)kXRanks; ++r)
        if (e->xchg_peers[r] && r != e->rank && !e->p2p_by_pointer) cudaIpcCloseMemHandle(e->xchg_peers[r] - kXDescWords);
    cudaFree(e->d_xchg);
    cudaFree(e->d_pipe_seg);
    cudaFree(e->d_log_seg_cnt);
    cudaFree(e->d_blk_prof);
    for (void* p : e->bk_arrays) cudaFree(p);
    cudaFree(e->d_bk_ctl);
    cudaFree(e->d_pipe_sync);
    cudaFree(e->d_log_keys); cudaFree(e->d_log_keys2); cudaFree(e->d_log_tmp);
    for (uint32_t* p : e->h_spk_blocks) cudaFreeHost(p);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
    return BMTK_OK;
}

int bmtk_engine_set_nodes(bmtk_engine* e, uint64_t n_global, uint64_t lo, uint64_t n_local, const uint16_t* type_index,
                          int32_t n_types, const bmtk_glif_params* types) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "set_nodes: engine missing or already finalized");
    if (n_types < 1 || n_types > 65535 || !types) return fail(BMTK_E_INVALID, "set_nodes: need 1..65535 node types");
    if (lo + n_local > n_global) return fail(BMTK_E_INVALID, "set_nodes: block [%llu,%llu) outside 0..%llu",
                                             (unsigned long long)lo, (unsigned long long)(lo + n_local),
                                             (unsigned long long)n_global);
    if (n_local && !type_index) return fail(BMTK_E_INVALID, "set_nodes: type_index is NULL");
    if (n_global >= (1ull << kSrcBits)) return fail(BMTK_E_UNSUPPORTED, "more than 2^%d sources", kSrcBits);
    for (uint64_t i = 0; i < n_local; ++i)
        if (type_index[i] >= n_types) return fail(BMTK_E_INVALID, "set_nodes: type_index[%llu] out of range", (unsigned long long)i);
    TypeConsts tmp;
    for (int t = 0; t < n_types; ++t) {
        const int rc = compute_type_consts(types[t], e->dt, tmp);
        if (rc) return rc;
    }
    e->n_global = n_global;
    e->lo = lo;
    e->n_local = n_local;
    e->type_index.assign(type_index, type_index + n_local);
    e->types.assign(types, types + n_types);
    e->has_theta = false;
    for (auto& t : e->types) e->has_theta |= (t.spike_dependent_threshold || t.adapting_threshold);
    return BMTK_OK;
}

int bmtk_engine_set_virtual(bmtk_engine* e, uint64_t n_virtual) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "set_virtual: engine missing or already finalized");
    if (e->n_global + n_virtual >= (1ull << kSrcBits)) return fail(BMTK_E_UNSUPPORTED, "more than 2^%d sources", kSrcBits);
    e->n_virtual = n_virtual;
    return BMTK_OK;
}

int bmtk_engine_add_edges(bmtk_engine* e, uint64_t n, const uint32_t* src, const uint32_t* trg, const float* weight,
                          const uint16_t* delay_steps, const uint8_t* port) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "add_edges: engine missing or already finalized");
    if (n == 0) return BMTK_OK;
    if (!src || !trg || !weight || !delay_steps || !port) return fail(BMTK_E_INVALID, "add_edges: NULL array");
    const uint64_t n_rows = e->n_global + e->n_virtual;
    for (uint64_t i = 0; i < n; ++i) {
        if (delay_steps[i] < 1)
            return fail(BMTK_E_DELAY, "edge %llu: delay shorter than the resolution dt = %g ms",
                        (unsigned long long)i, e->dt);
        if (src[i] >= n_rows) return fail(BMTK_E_INVALID, "edge %llu: source %u out of range", (unsigned long long)i, src[i]);
        if (trg[i] < e->lo || trg[i] >= e->lo + e->n_local)
            return fail(BMTK_E_INVALID, "edge %llu: target %u outside this engine's block", (unsigned long long)i, trg[i]);
        if (port[i] >= kPorts) return fail(BMTK_E_INVALID, "edge %llu: port %u out of range", (unsigned long long)i, port[i]);
    }
    e->e_src.insert(e->e_src.end(), src, src + n);
    e->e_trg.insert(e->e_trg.end(), trg, trg + n);
    e->e_w.insert(e->e_w.end(), weight, weight + n);
    e->e_delay.insert(e->e_delay.end(), delay_steps, delay_steps + n);
    e->e_port.insert(e->e_port.end(), port, port + n);
    return BMTK_OK;
}

int bmtk_engine_set_input_spikes(bmtk_engine* e, uint64_t n, const uint32_t* virt_index, const uint32_t* stamp_step) {
    if (!e) return fail(BMTK_E_INVALID, "engine is NULL");
    if (n && (!virt_index || !stamp_step)) return fail(BMTK_E_INVALID, "set_input_spikes: NULL array");
    if (e->finalized && e->n_trials > 1) return fail(BMTK_E_UNSUPPORTED, "trials > 1 take Poisson cells only");
    for (uint64_t i = 0; i < n; ++i) {
        if (virt_index[i] >= e->n_virtual)
            return fail(BMTK_E_INVALID, "input spike %llu: virtual cell %u out of range", (unsigned long long)i, virt_index[i]);
        if (stamp_step[i] < 1)
            return fail(BMTK_E_INVALID, "input spike %llu: spike time must be greater than zero", (unsigned long long)i);
    }
    e->pending_in_virt.assign(virt_index, virt_index + n);
    e->pending_in_stamp.assign(stamp_step, stamp_step + n);
    e->has_pending_inputs = true;
    return BMTK_OK;
}

int bmtk_engine_set_poisson(bmtk_engine* e, const float* rate_hz, uint64_t seed) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "set_poisson: engine missing or already finalized");
    if (!rate_hz || e->n_virtual == 0) return fail(BMTK_E_INVALID, "set_poisson: no virtual cells or NULL rates");
    for (uint64_t v = 0; v < e->n_virtual; ++v) {
        const double lam = (double)rate_hz[v] * e->dt * 1e-3;
        if (!(lam >= 0) || lam > 0.25)
            return fail(BMTK_E_UNSUPPORTED, "virtual cell %llu: rate*dt = %g outside [0, 0.25]", (unsigned long long)v, lam);
    }
    e->poisson_rates.assign(rate_hz, rate_hz + e->n_virtual);
    e->seed = seed;
    e->has_poisson = true;
    return BMTK_OK;
}

int bmtk_engine_set_clamp_events(bmtk_engine* e, uint64_t n, const uint64_t* step, const uint32_t* target,
                                 const float* delta_pA) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "set_clamp_events: engine missing or already finalized");
    if (n && (!step || !target || !delta_pA)) return fail(BMTK_E_INVALID, "set_clamp_events: NULL array");
    for (uint64_t i = 0; i < n; ++i)
        if (target[i] < e->lo || target[i] >= e->lo + e->n_local)
            return fail(BMTK_E_INVALID, "clamp event %llu: target %u outside this engine's block", (unsigned long long)i, target[i]);
    e->ce_step_in.assign(step, step + n);
    e->ce_target_in.assign(target, target + n);
    e->ce_delta_in.assign(delta_pA, delta_pA + n);
    e->has_iext = n > 0;
    return BMTK_OK;
}

int bmtk_engine_record_spikes(bmtk_engine* e, int enable) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "record_spikes: engine missing or already finalized");
    e->record_spikes = enable != 0;
    return BMTK_OK;
}

int bmtk_engine_record_state(bmtk_engine* e, uint64_t n_ids, const uint32_t* ids, uint32_t interval_steps, int32_t n_vars,
                             const int32_t* vars) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "record_state: engine missing or already finalized");
    if (n_vars < 1 || n_vars > 8 || !vars) return fail(BMTK_E_INVALID, "record_state: 1..8 variables");
    uint32_t packed = 0;
    for (int32_t v = 0; v < n_vars; ++v) {
        if (vars[v] < 0 || vars[v] > BMTK_VAR_I) return fail(BMTK_E_INVALID, "record_state: unknown variable code %d", vars[v]);
        packed |= (uint32_t)vars[v] << (4 * v);
    }
    const int rc = bmtk_engine_record_vm(e, n_ids, ids, interval_steps);
    if (rc) return rc;
    e->n_probe_vars = (uint32_t)n_vars;
    e->probe_vars = packed;
    return BMTK_OK;
}

int bmtk_engine_record_vm(bmtk_engine* e, uint64_t n_ids, const uint32_t* ids, uint32_t interval_steps) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "record_vm: engine missing or already finalized");
    if (interval_steps < 1) return fail(BMTK_E_INVALID, "record_vm: interval must be at least one step");
    const uint64_t span = e->n_trials > 1 ? (uint64_t)e->n_trials * ((e->n_local + 3) / 4 * 4) : e->n_local;
    for (uint64_t i = 0; i < n_ids; ++i)
        if (ids[i] < e->lo || ids[i] >= e->lo + span)
            return fail(BMTK_E_INVALID, "record_vm: id %u outside this engine's block", ids[i]);
    e->probe_ids.resize(n_ids);
    for (uint64_t i = 0; i < n_ids; ++i) e->probe_ids[i] = ids[i] - (uint32_t)e->lo;
    e->probe_interval = interval_steps;
    e->n_probe_vars = 1;
    e->probe_vars = BMTK_VAR_V_M;
    return BMTK_OK;
}

int bmtk_engine_set_option(bmtk_engine* e, const char* key, int64_t value) {
    if (!e || !key) return fail(BMTK_E_INVALID, "set_option: NULL argument");
    const std::string k(key);
    if (k == "profile") { e->profile = value != 0; return BMTK_OK; }
    if (k == "use_graph") { e->use_graph = value != 0; return BMTK_OK; }
    if (k == "persistent") { e->persistent = value != 0; return BMTK_OK; }
    if (k == "spike_store_reserve") {
        // pin host blocks for this many recorded spikes now rather than as they arrive
        constexpr size_t B = bmtk_engine::kSpkBlock;
        if (value < 0 || (uint64_t)value > (1ull << 34)) return fail(BMTK_E_INVALID, "spike_store_reserve out of range");
        int rc = set_device(e);
        if (rc) return rc;
        while (e->h_spk_blocks.size() * B < (uint64_t)value) {
            uint32_t* p = nullptr;
            CU(cudaMallocHost(&p, 4 * 2 * B));
            e->h_spk_blocks.push_back(p);
        }
        return BMTK_OK;
    }
    if (k == "pipeline") {
        if (e->finalized && e->n_ranks > 1)
            return fail(BMTK_E_INVALID, "with several ranks option 'pipeline' must be set before finalize (the ranks agree on the kernel when they connect)");
        e->pipeline = value != 0;
        return BMTK_OK;
    }
    if (k == "phase_timers") { e->phase_timers = value != 0; return BMTK_OK; }
    if (k == "replay_on_overflow") { e->replay = value != 0; return BMTK_OK; }
    if (k == "ring_prefetch") { e->ring_prefetch = value != 0; return BMTK_OK; }
    if (k == "ring_stage") { e->ring_stage = value != 0; return BMTK_OK; }
    if (k == "pipeline_warps") {
        if (value != 0 && value != (long long)pipelined_warps() && value != (long long)pipelined_warps_small())
            return fail(BMTK_E_INVALID, "pipeline_warps is 0 (choose), %u or %u", pipelined_warps_small(), pipelined_warps());
        if (e->finalized && e->n_ranks > 1)
            return fail(BMTK_E_INVALID, "with several ranks option 'pipeline_warps' must be set before finalize");
        e->pipe_warps_opt = (uint32_t)value;
        return BMTK_OK;
    }
    if (k == "tune") { e->tune = (uint32_t)value; return BMTK_OK; }
    if (k == "chunk_steps") {
        if (value < 1) return fail(BMTK_E_INVALID, "chunk_steps must be positive");
        e->chunk_steps = (uint64_t)value;
        return BMTK_OK;
    }
    if (e->finalized) return fail(BMTK_E_INVALID, "option '%s' must be set before finalize", key);
    if (value < 0) return fail(BMTK_E_INVALID, "option '%s' must not be negative", key);
    if (k == "deterministic") e->deterministic = value != 0;
    else if (k == "trials") {
        if (value < 1 || value > 4096) return fail(BMTK_E_INVALID, "trials must be 1..4096");
        e->n_trials = (uint32_t)value;
    }
    else if (k == "trial_base") e->trial_base = (uint32_t)value;
    else if (k == "window") e->window_opt = (uint32_t)value;
    else if (k == "pipeline_blocks") e->pipe_blocks_opt = (uint32_t)value;
    else if (k == "pipeline_trials") e->pipe_trials_opt = (uint32_t)value;
    else if (k == "spike_capacity") e->spike_cap_opt = (uint64_t)value;
    else if (k == "log_capacity") e->log_cap = std::max<uint64_t>(1024, (uint64_t)value);
    else if (k == "event_capacity") e->event_cap = std::max<uint64_t>(1024, (uint64_t)value);
    else return fail(BMTK_E_INVALID, "unknown option '%s'", key);
    return BMTK_OK;
}

int bmtk_comm_unique_id(void* uid128, const char* libnccl) {
    if (!uid128) return fail(BMTK_E_INVALID, "uid128 is NULL");
    int rc = load_nccl(libnccl);
    if (rc) return rc;
    Uid id;
    std::memset(&id, 0, sizeof(id));
    rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return fail(BMTK_E_COMM, "ncclGetUniqueId failed (%d)", rc);
    std::memcpy(uid128, &id, sizeof(id));
    return BMTK_OK;
}

int bmtk_engine_comm_init(bmtk_engine* e, const void* uid128, int rank, int n_ranks, const char* libnccl) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "comm_init: engine missing or already finalized");
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(BMTK_E_INVALID, "comm_init: bad rank %d of %d", rank, n_ranks);
    if (n_ranks > 16) return fail(BMTK_E_UNSUPPORTED, "at most 16 ranks");
    e->rank = rank;
    e->n_ranks = n_ranks;
    if (n_ranks == 1) return BMTK_OK;
    if (!uid128) return BMTK_OK;   // no NCCL communicator: only the peer-memory exchange can be used
    int rc = load_nccl(libnccl);
    if (rc) return rc;
    rc = set_device(e);
    if (rc) return rc;
    Uid id;
    std::memcpy(&id, uid128, sizeof(id));
    rc = g_nccl.CommInitRank(&e->comm, n_ranks, id, rank);
    if (rc != 0) return fail(BMTK_E_COMM, "ncclCommInitRank failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
    return BMTK_OK;
}

int bmtk_engine_finalize(bmtk_engine* e) {
    if (!e || e->finalized) return fail(BMTK_E_INVALID, "finalize: engine missing or already finalized");
    if (e->types.empty()) return fail(BMTK_E_INVALID, "finalize: set_nodes has not been called");
    int rc = set_device(e);
    if (rc) return rc;
    const uint64_t n_rows = e->n_global + e->n_virtual;
    e->n_edges = e->e_src.size();
    e->n_pad1 = (uint32_t)((e->n_local + 3) / 4 * 4);
    if (e->n_pad1 == 0) e->n_pad1 = 4;
    if (e->n_trials > 1) {
        if (e->n_ranks > 1 || e->lo != 0 || e->n_local != e->n_global)
            return fail(BMTK_E_UNSUPPORTED, "trials > 1 need the whole network on one rank (shard the trials over ranks instead)");
        if (e->deterministic) return fail(BMTK_E_UNSUPPORTED, "trials > 1 are not available with deterministic delivery");
        if (e->has_pending_inputs || !e->ce_step_in.empty())
            return fail(BMTK_E_UNSUPPORTED, "trials > 1 take Poisson cells only (no replayed spikes, no clamps)");
        if ((uint64_t)e->n_trials * (e->n_pad1 + e->n_virtual) >= (1ull << kSrcBits))
            return fail(BMTK_E_UNSUPPORTED, "trials x (neurons + virtual cells) exceeds 2^%d source ids", kSrcBits);
    }
    e->n_pad = e->n_pad1 * e->n_trials;

    // delays and the bit layout of a CSR entry
    uint32_t dmax = 1, dmin = 0xffffffffu;
    for (uint16_t d : e->e_delay) {
        dmax = std::max<uint32_t>(dmax, d);
        dmin = std::min<uint32_t>(dmin, d);
    }
    if (e->n_edges == 0) dmin = kMaxWindow;
    e->max_delay = dmax;
    e->min_delay = dmin;
    if (e->g_layout_set) {
        if (e->n_edges && e->g_min_delay > dmin)
            return fail(BMTK_E_INVALID, "set_global_layout: minimum delay %llu exceeds this rank's own minimum %u",
                        (unsigned long long)e->g_min_delay, dmin);
        if (e->g_max_local < e->n_local)
            return fail(BMTK_E_INVALID, "set_global_layout: largest block %llu is smaller than this rank's %llu neurons",
                        (unsigned long long)e->g_max_local, (unsigned long long)e->n_local);
        dmin = (uint32_t)std::min<uint64_t>(e->g_min_delay ? e->g_min_delay : dmin, kMaxWindow);
    }
    uint32_t tb = 1;
    while ((1ull << tb) < e->n_pad1) ++tb;
    uint32_t db = 1;
    while ((1u << db) <= dmax) ++db;
    if (tb + 2 + db > 32)
        return fail(BMTK_E_UNSUPPORTED, "CSR entry needs %u target + 2 port + %u delay bits > 32", tb, db);
    e->target_bits = tb;

    // exchange window: at most the minimum delay (every spike of a window lands in a later one)
    uint32_t w = e->window_opt ? e->window_opt : dmin;
    w = std::min<uint32_t>(w, dmin);
    w = std::min<uint32_t>(w, kMaxWindow);
    w = std::max<uint32_t>(w, 1);
    e->window = w;
    e->ring_slots = dmax + w;
    const uint64_t ring_cells = (uint64_t)e->ring_slots * kPorts * e->n_pad;
    if (ring_cells >= (1ull << 32) && e->deterministic)
        return fail(BMTK_E_UNSUPPORTED, "deterministic mode needs fewer than 2^32 ring cells");

    // CSR
    rc = BMTK_OK;
    {
        cudaError_t ce = build_csr_device(n_rows, e->n_edges, e->e_src.data(), e->e_trg.data(), e->e_w.data(),
                                          e->e_delay.data(), e->e_port.data(), (uint32_t)e->lo, tb, e->stream,
                                          &e->d_rowptr, &e->d_entries);
        if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "CSR build failed: %s", cudaGetErrorString(ce));
    }
    std::vector<uint32_t>().swap(e->e_src);
    std::vector<uint32_t>().swap(e->e_trg);
    std::vector<float>().swap(e->e_w);
    std::vector<uint16_t>().swap(e->e_delay);
    std::vector<uint8_t>().swap(e->e_port);

    // state
    const size_t np = e->n_pad;
    CU(cudaMalloc(&e->st.U, 4 * np));
    CU(cudaMalloc(&e->st.asc0, 4 * np));
    CU(cudaMalloc(&e->st.asc1, 4 * np));
    CU(cudaMalloc(&e->st.y1, 4 * np * kPorts));
    CU(cudaMalloc(&e->st.y2, 4 * np * kPorts));
    CU(cudaMalloc(&e->st.refr, 4 * np));
    if (e->has_theta) {
        CU(cudaMalloc(&e->st.th_spike, 4 * np));
        CU(cudaMalloc(&e->st.th_voltage, 4 * np));
    }
    if (e->has_iext) CU(cudaMalloc(&e->st.i_ext, 4 * np));
    CU(cudaMalloc(&e->d_type, 2 * np));
    {
        std::vector<uint16_t> ty(np, 0);
        for (uint32_t t = 0; t < e->n_trials; ++t)      // every trial has the same cells
            std::copy(e->type_index.begin(), e->type_index.end(), ty.begin() + (size_t)t * e->n_pad1);
        CU(cudaMemcpy(e->d_type, ty.data(), 2 * np, cudaMemcpyHostToDevice));
    }
    e->st.type = e->d_type;
    const size_t nt = e->types.size();
    std::vector<TypeConsts> tc(nt);
    std::vector<float> init(nt * 3);
    for (size_t t = 0; t < nt; ++t) {
        rc = compute_type_consts(e->types[t], e->dt, tc[t]);
        if (rc) return rc;
        init[t * 3 + 0] = (float)(e->types[t].V_m - e->types[t].E_L);
        init[t * 3 + 1] = (float)e->types[t].asc_init[0];
        init[t * 3 + 2] = (float)e->types[t].asc_init[1];
    }
    CU(cudaMalloc(&e->d_types, sizeof(TypeConsts) * nt));
    CU(cudaMemcpy(e->d_types, tc.data(), sizeof(TypeConsts) * nt, cudaMemcpyHostToDevice));
    float* d_init = nullptr;
    CU(cudaMalloc(&d_init, 4 * init.size()));
    CU(cudaMemcpy(d_init, init.data(), 4 * init.size(), cudaMemcpyHostToDevice));
    init_state_kernel<<<(unsigned)((np + 255) / 256), 256, 0, e->stream>>>(e->st, e->d_types, d_init, e->n_pad);
    CU(cudaGetLastError());
    CU(cudaMalloc(&e->ring, 4 * ring_cells));
    CU(cudaMemsetAsync(e->ring, 0, 4 * ring_cells, e->stream));
    CU(cudaMalloc(&e->d_ctl, sizeof(Ctl)));
    CU(cudaMemsetAsync(e->d_ctl, 0, sizeof(Ctl), e->stream));
    CU(cudaStreamSynchronize(e->stream));
    cudaFree(d_init);

    // spike lists. Automatic capacity: every local neuron may fire in 1 of 8 steps of a window.
    const uint64_t n_cells = (e->g_layout_set ? e->g_max_local : (uint64_t)e->n_local) * e->n_trials;
    uint64_t cap = e->spike_cap_opt ? e->spike_cap_opt : std::max<uint64_t>(4096, n_cells * w / 8);
    cap = std::min<uint64_t>(cap, n_cells * w + 4);
    cap = (cap + 3) / 4 * 4;
    if (cap + 4 >= (1ull << 31)) return fail(BMTK_E_UNSUPPORTED, "spike_capacity too large");
    e->send_cap = (uint32_t)cap;
    const size_t seg = (size_t)e->send_cap + 4;  // word 0 = count, 3 words of padding keep 16-byte alignment
    CU(cudaMalloc(&e->d_send, 4 * seg));
    CU(cudaMemset(e->d_send, 0, 4 * seg));
    if (e->n_ranks > 1) {
        CU(cudaMalloc(&e->d_gathered, 4 * seg * e->n_ranks));
        CU(cudaMemset(e->d_gathered, 0, 4 * seg * e->n_ranks));
    }
    if (e->has_poisson) {
        uint64_t vc = e->spike_cap_opt ? e->spike_cap_opt : std::max<uint64_t>(4096, e->n_virtual * e->n_trials * w / 4);
        e->virt_cap = (uint32_t)vc;
        CU(cudaMalloc(&e->d_virt, 4 * ((size_t)e->virt_cap + 4)));
        CU(cudaMemset(e->d_virt, 0, 4 * ((size_t)e->virt_cap + 4)));
        std::vector<uint4> thr(e->n_virtual);
        for (uint64_t v = 0; v < e->n_virtual; ++v) {
            const double lam = (double)e->poisson_rates[v] * e->dt * 1e-3;
            double p = std::exp(-lam), cdf = 0.0;
            uint32_t t[4];
            for (int k = 0; k < 4; ++k) {
                cdf += p;
                const double x = std::floor(cdf * 4294967296.0);
                t[k] = x >= 4294967295.0 ? 0xFFFFFFFFu : (uint32_t)x;
                p *= lam / (double)(k + 1);
            }
            thr[v] = make_uint4(t[0], t[1], t[2], t[3]);
        }
        CU(cudaMalloc(&e->d_poisson_thr, sizeof(uint4) * e->n_virtual));
        CU(cudaMemcpy(e->d_poisson_thr, thr.data(), sizeof(uint4) * e->n_virtual, cudaMemcpyHostToDevice));
    }
    if (e->record_spikes) {
        if (e->log_cap >= (1ull << 32)) return fail(BMTK_E_UNSUPPORTED, "log_capacity too large");
        CU(cudaMalloc(&e->d_log_stamp, 4 * e->log_cap));
        CU(cudaMalloc(&e->d_log_id, 4 * e->log_cap));
        CU(cudaMalloc(&e->d_log_keys, 8 * e->log_cap));
        CU(cudaMalloc(&e->d_log_keys2, 8 * e->log_cap));
        e->log_tmp_bytes = spike_log_sort_tmp_bytes((uint32_t)e->log_cap);
        CU(cudaMalloc(&e->d_log_tmp, e->log_tmp_bytes));
    }
    // clamps: sort by step
    if (e->has_iext) {
        const size_t n = e->ce_step_in.size();
        std::vector<size_t> ord(n);
        for (size_t i = 0; i < n; ++i) ord[i] = i;
        std::stable_sort(ord.begin(), ord.end(), [&](size_t a, size_t b) { return e->ce_step_in[a] < e->ce_step_in[b]; });
        std::vector<uint32_t> tg(n);
        std::vector<float> dl(n);
        e->ce_step.resize(n);
        for (size_t i = 0; i < n; ++i) {
            e->ce_step[i] = e->ce_step_in[ord[i]];
            tg[i] = e->ce_target_in[ord[i]];
            dl[i] = e->ce_delta_in[ord[i]];
        }
        CU(cudaMalloc(&e->d_ce_target, 4 * n));
        CU(cudaMalloc(&e->d_ce_delta, 4 * n));
        CU(cudaMemcpy(e->d_ce_target, tg.data(), 4 * n, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(e->d_ce_delta, dl.data(), 4 * n, cudaMemcpyHostToDevice));
    }
    // probes
    if (!e->probe_ids.empty()) {
        const size_t n_ids = e->probe_ids.size(), n_vals = n_ids * e->n_probe_vars;
        // at most 256 MiB of trace between drains, at least 64 samples
        uint64_t cap_s = std::max<uint64_t>(64, (256ull << 20) / (4 * n_vals));
        cap_s = std::min<uint64_t>(cap_s, 1u << 20);
        e->trace_cap = (uint32_t)cap_s;
        CU(cudaMalloc(&e->d_probe_ids, 4 * n_ids));
        CU(cudaMemcpy(e->d_probe_ids, e->probe_ids.data(), 4 * n_ids, cudaMemcpyHostToDevice));
        CU(cudaMalloc(&e->d_trace, 4 * n_vals * cap_s));
    }
    // persistent stepping: second spike lists, clamp groups, probe map, grid size
    {
        if (e->has_poisson) {
            CU(cudaMalloc(&e->d_virt2, 4 * ((size_t)e->virt_cap + 4)));
            CU(cudaMemset(e->d_virt2, 0, 4 * ((size_t)e->virt_cap + 4)));
        }
        if (e->has_iext) {
            std::vector<unsigned long long> gs;
            std::vector<uint32_t> gp;
            for (size_t i = 0; i < e->ce_step.size(); ++i) {
                if (i == 0 || e->ce_step[i] != e->ce_step[i - 1]) {
                    gs.push_back(e->ce_step[i]);
                    gp.push_back((uint32_t)i);
                }
            }
            gp.push_back((uint32_t)e->ce_step.size());
            e->ce_group_step.assign(gs.begin(), gs.end());
            CU(cudaMalloc(&e->d_ce_group_step, 8 * std::max<size_t>(gs.size(), 1)));
            CU(cudaMalloc(&e->d_ce_group_ptr, 4 * gp.size()));
            if (!gs.empty()) CU(cudaMemcpy(e->d_ce_group_step, gs.data(), 8 * gs.size(), cudaMemcpyHostToDevice));
            CU(cudaMemcpy(e->d_ce_group_ptr, gp.data(), 4 * gp.size(), cudaMemcpyHostToDevice));
        }
        if (!e->probe_ids.empty()) {
            std::vector<int32_t> slot(np, -1);
            for (size_t q = 0; q < e->probe_ids.size(); ++q) slot[e->probe_ids[q]] = (int32_t)q;
            CU(cudaMalloc(&e->d_probe_slot, 4 * np));
            CU(cudaMemcpy(e->d_probe_slot, slot.data(), 4 * np, cudaMemcpyHostToDevice));
        }
        const size_t smem = persistent_smem((int)nt);
        const int blocks = persistent_max_blocks(e->device, e->has_theta, e->has_iext, true, smem);
        e->persist_blocks = blocks;
        if (blocks > 0) {
            const uint64_t gpb = (((uint64_t)(e->n_pad / 4) + blocks - 1) / blocks + 31) / 32 * 32;
            e->persist_resident = gpb <= persistent_threads_per_block();
        }
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, e->device);
        if (!coop || blocks > 512) e->persist_blocks = 0;
        if (e->persist_blocks > 0 && e->n_trials <= 4096 && e->ring_slots < (1u << 20) && e->window >= 2 &&
            e->n_edges < (1ull << 32)) {
            int pb = pipelined_max_blocks(e->device, e->has_theta, e->has_iext, pipelined_smem((int)nt, pipelined_warps() - 2u));   // the most a block can need (one update, one input warp)
            if (pb > 0 && e->pipe_blocks_opt) pb = std::min<int>(pb, (int)e->pipe_blocks_opt);
            if (pb > 0 && pb <= (int)kPipeMaxBlocks) {
                // chunks of 32 groups are dealt round-robin to the update warps of the blocks
                const uint64_t chunks1 = ((uint64_t)(e->n_pad1 / 4) + 31) / 32;   // of one trial
                // trials per launch (option pipeline_trials overrides): as many as the 12-warp block takes (no register
                // spills, packed arithmetic: measured 8 % ahead of three trials in the 20-warp block on 50 000 neurons);
                // where not even one trial fits that block, as many as leave three of the 20 warps to the delivering
                // side. Either way the ring slots of a launch stay within ~3/4 of L2.
                e->pipe_trials = 1;
                if (e->n_trials > 1) {
                    int l2 = 0;
                    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, e->device);
                    const uint64_t ring1 = (uint64_t)e->ring_slots * kPorts * e->n_pad1 * 4;
                    auto upd_warps_of = [&](uint32_t t) { return (uint32_t)((chunks1 * t + pb - 1) / pb); };
                    auto input_warps_of = [&](uint32_t t) {
                        return e->has_poisson ? std::max<uint32_t>(1, (uint32_t)((e->n_virtual * t / pb + 63) / 64)) : 1u;
                    };
                    auto fits_small = [&](uint32_t t) { return upd_warps_of(t) + input_warps_of(t) + 5u <= pipelined_warps_small(); };
                    auto fits_big = [&](uint32_t t) { return upd_warps_of(t) <= pipelined_max_update_warps() - 3u; };
                    const bool small = fits_small(1);
                    uint32_t t = 1;
                    while (t < e->n_trials && (small ? fits_small(t + 1) : fits_big(t + 1)) && ring1 * (t + 1) <= (uint64_t)l2 / 4 * 3)
                        ++t;
                    if (e->pipe_trials_opt) t = std::min<uint32_t>(e->pipe_trials_opt, e->n_trials);
                    e->pipe_trials = t;
                }
                const uint64_t chunks = chunks1 * e->pipe_trials;
                e->pipe_upd_warps = (uint32_t)std::max<uint64_t>(1, (chunks + pb - 1) / pb);
                e->pipe_ok = e->pipe_upd_warps <= pipelined_max_update_warps();
                e->pipe_blocks = pb;
                if (e->has_poisson) {
                    // a block adds its share of the Poisson spikes to its segment of the phase list: leave half for neurons
                    double lam = 0.0;
                    for (uint64_t v = 0; v < e->n_virtual; ++v) lam += (double)e->poisson_rates[v] * e->dt * 1e-3;
                    const double per_block = lam * e->pipe_trials * (e->window / 2) / pb;
                    if (per_block * 4.0 + 64.0 > (double)kPipeSegCap / 2) e->pipe_ok = false;
                }
                if (e->pipe_ok) {
                    CU(cudaMalloc(&e->d_pipe_seg, sizeof(uint4) * 3 * (size_t)pb * kPipeSegCap));
                    CU(cudaMalloc(&e->d_pipe_sync, 32));
                    CU(cudaMalloc(&e->d_blk_prof, 32 * (size_t)pb + 8 * 160 + 128 * (size_t)pb));
                    CU(cudaMemset(e->d_blk_prof, 0, 32 * (size_t)pb + 8 * 160 + 128 * (size_t)pb));
                    CU(cudaMalloc(&e->d_log_seg_cnt, 4 * (size_t)pb));
                    CU(cudaMemset(e->d_log_seg_cnt, 0, 4 * (size_t)pb));
                    // a descriptor is valid by its tag (first step of its phase + 1): none is at rest
                    CU(cudaMemset(e->d_pipe_seg, 0, sizeof(uint4) * 3 * (size_t)pb * kPipeSegCap));
                }
            }
        }
        if (e->persist_blocks > 0) {
            for (int q = 0; q < 2; ++q) CU(cudaMalloc(&e->d_plists[q], sizeof(uint4) * (size_t)e->send_cap));
            CU(cudaMalloc(&e->d_plist_counts, 8));
            CU(cudaMemset(e->d_plist_counts, 0, 8));
            if (e->n_ranks > 1) {
                // two-phase area, then the pipelined kernel's area (64-bit words each)
                const size_t words = xchg_words((uint32_t)e->n_ranks, e->send_cap);
                const size_t pwords = xpipe_words((uint32_t)e->n_ranks, (uint32_t)std::max(e->persist_blocks, e->pipe_blocks));
                e->xp_off = (uint32_t)words;
                // [layout descriptor | two-phase area | pipelined area]; kernels see the buffer from the two-phase area on
                CU(cudaMalloc(&e->d_xchg, 8 * (kXDescWords + words + pwords)));
                CU(cudaMemset(e->d_xchg, 0, 8 * (kXDescWords + words + pwords)));
                uint64_t desc[kXDescWords];
                describe_layout(e, desc);
                CU(cudaMemcpy(e->d_xchg, desc, sizeof(desc), cudaMemcpyHostToDevice));
            }
        }
    }
    if (e->deterministic) {
        cudaError_t ce = det_alloc(e->det, (uint32_t)e->event_cap,
                                   (uint32_t)((size_t)e->send_cap * e->n_ranks + e->virt_cap + 65536), ring_cells);
        if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "deterministic workspace: %s", cudaGetErrorString(ce));
    }
    if (e->comm) {
        // the ranks must agree on window and capacity before the first all-gather of spike lists: a
        // mismatch there would hang the collective, here it is one small all-gather and a clear error
        uint64_t desc[kXDescWords];
        describe_layout(e, desc);
        unsigned long long *d_mine = nullptr, *d_all = nullptr;
        CU(cudaMalloc(&d_mine, sizeof(desc)));
        CU(cudaMalloc(&d_all, sizeof(desc) * e->n_ranks));
        CU(cudaMemcpy(d_mine, desc, sizeof(desc), cudaMemcpyHostToDevice));
        const int nrc = g_nccl.AllGather(d_mine, d_all, 2 * kXDescWords, kNcclUint32, e->comm, e->stream);
        std::vector<uint64_t> all((size_t)kXDescWords * e->n_ranks);
        cudaError_t ce = nrc == 0 ? cudaStreamSynchronize(e->stream) : cudaSuccess;
        if (nrc == 0 && ce == cudaSuccess) ce = cudaMemcpy(all.data(), d_all, 8 * all.size(), cudaMemcpyDeviceToHost);
        cudaFree(d_mine);
        cudaFree(d_all);
        if (nrc != 0) return fail(BMTK_E_COMM, "ncclAllGather of the exchange layout failed: %s",
                                  g_nccl.GetErrorString ? g_nccl.GetErrorString(nrc) : "?");
        if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "exchange layout all-gather: %s", cudaGetErrorString(ce));
        for (int r = 0; r < e->n_ranks; ++r) {
            if (r == e->rank) continue;
            rc = compare_layout(desc, all.data() + (size_t)kXDescWords * r, r);
            if (rc) return rc;
        }
    }
    e->finalized = true;
    return BMTK_OK;
}

int bmtk_engine_local_layout(bmtk_engine* e, uint64_t* out4) {
    if (!e || !out4) return fail(BMTK_E_INVALID, "local_layout: NULL argument");
    uint64_t dmin = 0xffffffffull;
    for (uint16_t d : e->e_delay) dmin = std::min<uint64_t>(dmin, d);
    if (e->finalized) dmin = e->n_edges ? e->min_delay : 0xffffffffull;
    out4[0] = dmin;
    out4[1] = e->n_local;
    out4[2] = (e->has_iext || !e->ce_step_in.empty()) ? 1 : 0;
    out4[3] = 0;
    return BMTK_OK;
}

int bmtk_engine_set_global_layout(bmtk_engine* e, const uint64_t* in4) {
    if (!e || e->finalized || !in4) return fail(BMTK_E_INVALID, "set_global_layout: engine missing, already finalized, or NULL");
    if (in4[0] < 1) return fail(BMTK_E_INVALID, "set_global_layout: the minimum delay is at least one step");
    e->g_min_delay = in4[0];
    e->g_max_local = in4[1];
    e->g_any_clamps = in4[2] != 0;
    e->g_layout_set = true;
    return BMTK_OK;
}

int bmtk_engine_exchange_layout(bmtk_engine* e, uint64_t* out16) {
    if (!e || !e->finalized || !out16) return fail(BMTK_E_INVALID, "exchange_layout: engine missing, not finalized, or NULL");
    describe_layout(e, out16);
    return BMTK_OK;
}

int bmtk_exchange_layout_compare(const uint64_t* mine16, const uint64_t* theirs16, int their_rank) {
    if (!mine16 || !theirs16) return fail(BMTK_E_INVALID, "exchange_layout_compare: NULL argument");
    if (mine16[0] != kXDescMagic || theirs16[0] != kXDescMagic)
        return fail(BMTK_E_INVALID, "exchange_layout_compare: not a layout written by bmtk_engine_exchange_layout");
    return compare_layout(mine16, theirs16, their_rank);
}

int bmtk_engine_run(bmtk_engine* e, uint64_t n_steps) {
    if (!e || !e->finalized) return fail(BMTK_E_INVALID, "run: engine missing or not finalized");
    int rc = set_device(e);
    if (rc) return rc;
    if (e->step + n_steps >= (1ull << 32)) return fail(BMTK_E_UNSUPPORTED, "more than 2^32 steps");
    return run_steps(e, n_steps);
}

int bmtk_engine_spike_count(bmtk_engine* e, uint64_t* n) {
    if (!e || !n) return fail(BMTK_E_INVALID, "NULL argument");
    *n = e->h_spk_n;
    return BMTK_OK;
}

int bmtk_engine_fetch_spikes(bmtk_engine* e, uint64_t cap, uint32_t* stamp_step, uint32_t* id, uint64_t* n_out) {
    if (!e || !n_out) return fail(BMTK_E_INVALID, "NULL argument");
    const size_t n = e->h_spk_n;
    if (cap < n) return fail(BMTK_E_INVALID, "fetch_spikes: capacity %llu < %llu spikes", (unsigned long long)cap,
                             (unsigned long long)n);
    if (n && (!stamp_step || !id)) return fail(BMTK_E_INVALID, "fetch_spikes: NULL array");
    // already in canonical (stamp, id) order: sorted per chunk on the device, chunks consecutive in time
    constexpr size_t B = bmtk_engine::kSpkBlock;
    for (size_t done = 0; done < n; done += B) {
        const size_t take = std::min(n - done, B);
        std::memcpy(stamp_step + done, e->h_spk_blocks[done / B], 4 * take);
        std::memcpy(id + done, e->h_spk_blocks[done / B] + B, 4 * take);
    }
    *n_out = n;
    e->h_spk_n = 0;
    return BMTK_OK;
}

int bmtk_engine_trace_samples(bmtk_engine* e, uint64_t* n_samples) {
    if (!e || !n_samples) return fail(BMTK_E_INVALID, "NULL argument");
    *n_samples = e->probe_ids.empty() ? 0 : e->h_trace.size() / (e->probe_ids.size() * e->n_probe_vars);
    return BMTK_OK;
}

int bmtk_engine_fetch_trace(bmtk_engine* e, uint64_t cap_samples, float* vm, uint64_t* n_out) {
    if (!e || !n_out) return fail(BMTK_E_INVALID, "NULL argument");
    const size_t n_ids = e->probe_ids.size() * e->n_probe_vars;   // values per sample: [variable][id]
    const size_t n = n_ids ? e->h_trace.size() / n_ids : 0;
    if (cap_samples < n) return fail(BMTK_E_INVALID, "fetch_trace: capacity too small");
    if (n) std::memcpy(vm, e->h_trace.data(), 4 * n * n_ids);
    *n_out = n;
    e->h_trace.clear();
    return BMTK_OK;
}

int bmtk_engine_get_state(bmtk_engine* e, const char* var, float* out) {
    if (!e || !e->finalized || !var || !out) return fail(BMTK_E_INVALID, "get_state: bad argument");
    int rc = set_device(e);
    if (rc) return rc;
    const std::string v(var);
    // one trial: n_local values; several trials: all n_trials * n_pad1 cells (trial-major, padded)
    const size_t n = e->n_trials > 1 ? (size_t)e->n_pad : e->n_local, np = e->n_pad;
    const float* src = nullptr;
    if (v == "U" || v == "V_m") src = e->st.U;
    else if (v == "asc0") src = e->st.asc0;
    else if (v == "asc1") src = e->st.asc1;
    else if (v == "i_ext") src = e->st.i_ext;
    else if (v == "th_spike") src = e->st.th_spike;
    else if (v == "th_voltage") src = e->st.th_voltage;
    else if (v.size() == 4 && v[0] == 'y' && (v[1] == '1' || v[1] == '2') && v[2] == '_' && v[3] >= '0' && v[3] < '0' + kPorts)
        src = (v[1] == '1' ? e->st.y1 : e->st.y2) + (size_t)(v[3] - '0') * np;
    else if (v == "refr") {
        std::vector<int32_t> r(n);
        CU(cudaStreamSynchronize(e->stream));
        CU(cudaMemcpy(r.data(), e->st.refr, 4 * n, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n; ++i) out[i] = (float)r[i];
        return BMTK_OK;
    } else return fail(BMTK_E_INVALID, "get_state: unknown variable '%s'", var);
    if (!src) {
        for (size_t i = 0; i < n; ++i) out[i] = 0.f;
        return BMTK_OK;
    }
    CU(cudaStreamSynchronize(e->stream));
    CU(cudaMemcpy(out, src, 4 * n, cudaMemcpyDeviceToHost));
    if (v == "V_m")
        for (size_t i = 0; i < n; ++i) {
            const size_t c = i % e->n_pad1;
            if (c < e->n_local) out[i] += (float)e->types[e->type_index[c]].E_L;
        }
    return BMTK_OK;
}

int bmtk_engine_csr_info(bmtk_engine* e, uint64_t* n_rows, uint64_t* n_edges, uint32_t* target_bits, uint32_t* max_delay,
                         uint32_t* min_delay, uint32_t* ring_slots) {
    if (!e || !e->finalized) return fail(BMTK_E_INVALID, "csr_info: engine missing or not finalized");
    if (n_rows) *n_rows = e->n_global + e->n_virtual;
    if (n_edges) *n_edges = e->n_edges;
    if (target_bits) *target_bits = e->target_bits;
    if (max_delay) *max_delay = e->max_delay;
    if (min_delay) *min_delay = e->min_delay;
    if (ring_slots) *ring_slots = e->ring_slots;
    return BMTK_OK;
}

int bmtk_engine_get_csr(bmtk_engine* e, uint64_t* rowptr, uint32_t* packed, float* weight) {
    if (!e || !e->finalized) return fail(BMTK_E_INVALID, "get_csr: engine missing or not finalized");
    int rc = set_device(e);
    if (rc) return rc;
    const uint64_t n_rows = e->n_global + e->n_virtual;
    CU(cudaStreamSynchronize(e->stream));
    if (rowptr) CU(cudaMemcpy(rowptr, e->d_rowptr, 8 * (n_rows + 1), cudaMemcpyDeviceToHost));
    if ((packed || weight) && e->n_edges) {
        std::vector<uint2> h(e->n_edges);
        CU(cudaMemcpy(h.data(), e->d_entries, 8 * e->n_edges, cudaMemcpyDeviceToHost));
        for (uint64_t i = 0; i < e->n_edges; ++i) {
            if (packed) packed[i] = h[i].x;
            if (weight) std::memcpy(&weight[i], &h[i].y, 4);
        }
    }
    return BMTK_OK;
}

int bmtk_propagate_spikes(const uint64_t* d_rowptr, const void* d_entries, uint32_t target_bits, uint32_t n_spikes,
                          const uint32_t* d_spike_src, const uint32_t* d_spike_step, float* d_ring,
                          uint32_t ring_slots, uint32_t n_pad, int deterministic, void* stream) {
    if (!d_rowptr || !d_entries || !d_ring) return fail(BMTK_E_INVALID, "propagate_spikes: NULL device pointer");
    if (n_spikes && (!d_spike_src || !d_spike_step)) return fail(BMTK_E_INVALID, "propagate_spikes: NULL spike list");
    if (ring_slots < 1 || n_pad < 1 || target_bits < 1 || target_bits > 29)
        return fail(BMTK_E_INVALID, "propagate_spikes: bad ring geometry");
    if (n_spikes == 0) return BMTK_OK;
    cudaStream_t st = (cudaStream_t)stream;
    Ctl* d_ctl = nullptr;
    uint32_t* d_in_ptr = nullptr;
    CU(cudaMalloc(&d_ctl, sizeof(Ctl)));
    if (cudaMalloc(&d_in_ptr, 8) != cudaSuccess) {
        cudaFree(d_ctl);
        return fail(BMTK_E_CUDA, "propagate_spikes: cudaMalloc failed");
    }
    const uint32_t h_ptr[2] = {0u, n_spikes};
    int rc = BMTK_OK;
    DetWorkspace ws{};
    do {
        if (cudaMemsetAsync(d_ctl, 0, sizeof(Ctl), st) != cudaSuccess ||
            cudaMemcpyAsync(d_in_ptr, h_ptr, 8, cudaMemcpyHostToDevice, st) != cudaSuccess) {
            rc = fail(BMTK_E_CUDA, "propagate_spikes: set-up copy failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        PropArgs a{};
        a.rowptr = (const unsigned long long*)d_rowptr;
        a.entries = (const uint2*)d_entries;
        a.target_bits = target_bits;
        a.ring = d_ring;
        a.ring_slots = ring_slots;
        a.n_pad = n_pad;
        a.ctl = d_ctl;
        a.n_seg = 0;
        a.in_ptr = d_in_ptr;
        a.in_ptr_base = 0;
        a.in_ptr_len = 2;
        a.in_step = d_spike_step;
        a.in_src = d_spike_src;
        a.window = 1;
        if (deterministic) {
            const uint64_t cells = (uint64_t)ring_slots * kPorts * n_pad;
            if (cells >= (1ull << 32)) { rc = fail(BMTK_E_UNSUPPORTED, "propagate_spikes: ring too large"); break; }
            const uint32_t event_cap = 1u << 22;
            if (det_alloc(ws, event_cap, n_spikes, cells) != cudaSuccess) {
                rc = fail(BMTK_E_CUDA, "propagate_spikes: workspace allocation failed");
                break;
            }
            uint64_t launches = 0;
            const int r = propagate_det_window(a, ws, st, &launches);
            if (r == -2) { rc = fail(BMTK_E_OVERFLOW, "propagate_spikes: more than %u events in one call", event_cap); break; }
            if (r != 0) { rc = fail(BMTK_E_CUDA, "propagate_spikes: %s", cudaGetErrorString(cudaGetLastError())); break; }
        } else {
            if (launch_propagate_atomic(a, st) != cudaSuccess) {
                rc = fail(BMTK_E_CUDA, "propagate_spikes: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
                break;
            }
        }
        if (cudaStreamSynchronize(st) != cudaSuccess)
            rc = fail(BMTK_E_CUDA, "propagate_spikes: %s", cudaGetErrorString(cudaGetLastError()));
    } while (0);
    det_free(ws);
    cudaFree(d_ctl);
    cudaFree(d_in_ptr);
    return rc;
}

int bmtk_probe_scatter_reductions(int device, uint64_t n_cells, uint64_t n_ops, int repeats, double* ms_per_pass) {
    if (!ms_per_pass || n_cells < 1 || n_cells >= (1ull << 32) || n_ops < 1 || repeats < 1)
        return fail(BMTK_E_INVALID, "probe_scatter_reductions: bad argument");
    CU(cudaSetDevice(device));
    float* cells = nullptr;
    CU(cudaMalloc(&cells, 4 * n_cells));
    cudaEvent_t a = nullptr, b = nullptr;
    int rc = BMTK_OK;
    do {
        if (cudaMemset(cells, 0, 4 * n_cells) != cudaSuccess || cudaEventCreate(&a) != cudaSuccess ||
            cudaEventCreate(&b) != cudaSuccess) { rc = fail(BMTK_E_CUDA, "probe set-up failed"); break; }
        launch_scatter_red_probe(cells, (uint32_t)n_cells, n_ops, 0);   // warm-up
        cudaEventRecord(a, 0);
        for (int r = 0; r < repeats; ++r) launch_scatter_red_probe(cells, (uint32_t)n_cells, n_ops, 0);
        cudaEventRecord(b, 0);
        if (cudaEventSynchronize(b) != cudaSuccess) { rc = fail(BMTK_E_CUDA, "probe failed: %s", cudaGetErrorString(cudaGetLastError())); break; }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, a, b);
        *ms_per_pass = (double)ms / repeats;
    } while (0);
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    cudaFree(cells);
    return rc;
}

// ---- checkpoint / resume: the dynamic state is (step, neuron state arrays, ring buffer); Poisson
// cells are counter based and need none.
namespace {
struct CkptHeader {
    char magic[8];
    uint64_t step, n_global, lo, n_local;
    uint32_t n_pad, ring_slots, has_theta, has_iext;
    double dt;
};
}  // namespace

// Reads the layout descriptor at the head of every mapped exchange buffer and compares it with this
// rank's: a sender indexes the receiver's buffer with its OWN capacity and offsets, so a difference
// would put peer stores outside the receiver's allocation. Also settles what the ranks must decide
// together: the pipelined kernel only if every rank can run it and no rank has clamp changes.
static int check_peer_layouts(bmtk_engine* e) {
    uint64_t mine[kXDescWords], theirs[kXDescWords];
    describe_layout(e, mine);
    e->peers_pipe_ok = mine[7] != 0;
    e->any_iext = mine[8] != 0 || e->g_any_clamps;
    for (int r = 0; r < e->n_ranks; ++r) {
        if (r == e->rank) continue;
        CU(cudaMemcpy(theirs, e->xchg_peers[r] - kXDescWords, sizeof(theirs), cudaMemcpyDeviceToHost));
        if (theirs[0] != kXDescMagic)
            return fail(BMTK_E_COMM, "p2p_connect: the buffer of rank %d is not an exchange buffer of this library", r);
        const int rc = compare_layout(mine, theirs, r);
        if (rc) return rc;
        e->peers_pipe_ok = e->peers_pipe_ok && theirs[7] != 0;
        e->any_iext = e->any_iext || theirs[8] != 0;
    }
    return BMTK_OK;
}

int bmtk_engine_p2p_handle(bmtk_engine* e, void* handle64) {
    if (!e || !e->finalized || !handle64) return fail(BMTK_E_INVALID, "p2p_handle: engine missing, not finalized, or NULL");
    if (!e->d_xchg) return fail(BMTK_E_UNSUPPORTED, "p2p_handle: no exchange buffer (one rank, or cooperative launch unavailable)");
    int rc = set_device(e);
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    CU(cudaIpcGetMemHandle(&h, e->d_xchg));
    std::memcpy(handle64, &h, 64);
    return BMTK_OK;
}

int bmtk_engine_p2p_connect(bmtk_engine* e, const void* handles) {
    if (!e || !e->finalized || !handles) return fail(BMTK_E_INVALID, "p2p_connect: engine missing, not finalized, or NULL");
    if (!e->d_xchg) return fail(BMTK_E_UNSUPPORTED, "p2p_connect: no exchange buffer");
    int rc = set_device(e);
    if (rc) return rc;
    for (int r = 0; r < e->n_ranks; ++r) {
        if (r == e->rank) {
            e->xchg_peers[r] = e->d_xchg + kXDescWords;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const char*)handles + 64 * r, 64);
        void* p = nullptr;
        cudaError_t ce = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (ce != cudaSuccess)
            return fail(BMTK_E_COMM, "p2p_connect: cannot map the exchange buffer of rank %d: %s", r, cudaGetErrorString(ce));
        e->xchg_peers[r] = (unsigned long long*)p + kXDescWords;
    }
    rc = check_peer_layouts(e);
    if (rc) return rc;
    e->p2p_ready = true;
    return BMTK_OK;
}

// One thread per side bounces a tagged 8-byte word between two ranks' exchange buffers `rounds` times: plain peer
// store, polling load on the own buffer, the same primitives the stepping kernels exchange spikes with.
__global__ void pingpong_kernel(unsigned long long* my_inbox, unsigned long long* peer_inbox, int initiator, uint32_t rounds,
                                uint32_t base, unsigned long long* out_ns, uint32_t* timed_out) {
    unsigned long long t0 = 0ull;
    for (uint32_t i = 1; i <= rounds + 8u; ++i) {      // 8 untimed rounds first
        const uint32_t tag = base + i;
        if (i == 9u) t0 = gtimer();
        if (initiator) st_word(peer_inbox, tag, i);
        unsigned int spins = 0;
        while ((uint32_t)(ld_word(my_inbox) >> 32) != tag) {
            if (++spins > 40000000u) {   // a few seconds: the peer never answered
                *timed_out = 1u;
                return;
            }
        }
        if (!initiator) st_word(peer_inbox, tag, i);
    }
    *out_ns = gtimer() - t0;
}

int bmtk_engine_p2p_pingpong(bmtk_engine* e, int peer_rank, int initiator, uint32_t rounds, double* one_way_ns) {
    if (!e || !e->finalized || !one_way_ns) return fail(BMTK_E_INVALID, "p2p_pingpong: engine missing, not finalized, or NULL");
    if (!e->p2p_ready || peer_rank < 0 || peer_rank >= e->n_ranks || peer_rank == e->rank || rounds < 1)
        return fail(BMTK_E_INVALID, "p2p_pingpong: peers are not connected, or bad peer / round count");
    int rc = set_device(e);
    if (rc) return rc;
    unsigned long long* d_out = nullptr;
    CU(cudaMalloc(&d_out, 16));
    CU(cudaMemsetAsync(d_out, 0, 16, e->stream));
    // words 13 (ping) and 14 (pong) of the layout descriptor at the head of an exchange buffer are free for this
    unsigned long long* mine = e->d_xchg + (initiator ? 14 : 13);
    unsigned long long* theirs = e->xchg_peers[peer_rank] - kXDescWords + (initiator ? 13 : 14);
    e->pingpong_calls += 1;
    pingpong_kernel<<<1, 1, 0, e->stream>>>(mine, theirs, initiator, rounds, e->pingpong_calls << 20, d_out,
                                            reinterpret_cast<uint32_t*>(d_out + 1));
    unsigned long long h[2] = {0, 0};
    cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(h, d_out, 16, cudaMemcpyDeviceToHost, e->stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    cudaFree(d_out);
    if (ce != cudaSuccess) return fail(BMTK_E_CUDA, "p2p_pingpong: %s", cudaGetErrorString(ce));
    if ((uint32_t)h[1]) return fail(BMTK_E_COMM, "p2p_pingpong: rank %d did not answer within a few seconds", peer_rank);
    *one_way_ns = (double)h[0] / (2.0 * rounds);
    return BMTK_OK;
}

int bmtk_engine_p2p_buffer(bmtk_engine* e, void** d_buffer) {
    if (!e || !e->finalized || !d_buffer) return fail(BMTK_E_INVALID, "p2p_buffer: engine missing, not finalized, or NULL");
    if (!e->d_xchg) return fail(BMTK_E_UNSUPPORTED, "p2p_buffer: no exchange buffer (one rank, or cooperative launch unavailable)");
    *d_buffer = e->d_xchg;
    return BMTK_OK;
}

int bmtk_engine_p2p_connect_pointers(bmtk_engine* e, void* const* d_buffers) {
    if (!e || !e->finalized || !d_buffers) return fail(BMTK_E_INVALID, "p2p_connect_pointers: engine missing, not finalized, or NULL");
    if (!e->d_xchg) return fail(BMTK_E_UNSUPPORTED, "p2p_connect_pointers: no exchange buffer");
    for (int r = 0; r < e->n_ranks; ++r) {
        if (r != e->rank && !d_buffers[r]) return fail(BMTK_E_INVALID, "p2p_connect_pointers: buffer of rank %d is NULL", r);
        e->xchg_peers[r] = (r == e->rank ? e->d_xchg : (unsigned long long*)d_buffers[r]) + kXDescWords;
    }
    e->p2p_by_pointer = true;
    int rc = set_device(e);
    if (!rc) rc = check_peer_layouts(e);
    if (rc) return rc;
    e->p2p_ready = true;
    return BMTK_OK;
}

int bmtk_engine_save_state(bmtk_engine* e, const char* path) {
    if (!e || !e->finalized || !path) return fail(BMTK_E_INVALID, "save_state: engine missing, not finalized, or NULL path");
    int rc = set_device(e);
    if (rc) return rc;
    CU(cudaStreamSynchronize(e->stream));
    FILE* f = std::fopen(path, "wb");
    if (!f) return fail(BMTK_E_INVALID, "save_state: cannot open %s", path);
    CkptHeader h{};
    std::memcpy(h.magic, "BMTKB2C1", 8);
    h.step = e->step; h.n_global = e->n_global; h.lo = e->lo; h.n_local = e->n_local;
    h.n_pad = e->n_pad; h.ring_slots = e->ring_slots; h.has_theta = e->has_theta; h.has_iext = e->has_iext;
    h.dt = e->dt;
    bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1;
    std::vector<char> buf;
    for (const CkptArray& a : ckpt_arrays(e)) {
        if (!ok) break;
        buf.resize(a.bytes);
        if (cudaMemcpy(buf.data(), a.dev, a.bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = false; break; }
        ok = std::fwrite(buf.data(), 1, a.bytes, f) == a.bytes;
    }
    std::fclose(f);
    if (!ok) return fail(BMTK_E_CUDA, "save_state: writing %s failed", path);
    return BMTK_OK;
}

int bmtk_engine_load_state(bmtk_engine* e, const char* path) {
    if (!e || !e->finalized || !path) return fail(BMTK_E_INVALID, "load_state: engine missing, not finalized, or NULL path");
    int rc = set_device(e);
    if (rc) return rc;
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(BMTK_E_INVALID, "load_state: cannot open %s", path);
    CkptHeader h{};
    if (std::fread(&h, sizeof(h), 1, f) != 1 || std::memcmp(h.magic, "BMTKB2C1", 8) != 0) {
        std::fclose(f);
        return fail(BMTK_E_INVALID, "load_state: %s is not a bmtk_b200 checkpoint", path);
    }
    if (h.n_global != e->n_global || h.lo != e->lo || h.n_local != e->n_local || h.n_pad != e->n_pad ||
        h.ring_slots != e->ring_slots || h.has_theta != (uint32_t)e->has_theta || h.has_iext != (uint32_t)e->has_iext ||
        h.dt != e->dt) {
        std::fclose(f);
        return fail(BMTK_E_INVALID, "load_state: checkpoint was written for a different network, partition or dt");
    }
    CU(cudaStreamSynchronize(e->stream));
    std::vector<char> buf;
    bool ok = true;
    for (const CkptArray& a : ckpt_arrays(e)) {
        buf.resize(a.bytes);
        if (std::fread(buf.data(), 1, a.bytes, f) != a.bytes) { ok = false; break; }
        if (cudaMemcpy(a.dev, buf.data(), a.bytes, cudaMemcpyHostToDevice) != cudaSuccess) { ok = false; break; }
    }
    std::fclose(f);
    if (!ok) return fail(BMTK_E_CUDA, "load_state: reading %s failed", path);
    e->step = h.step;
    const unsigned long long sb = h.step;
    CU(cudaMemcpy(&e->d_ctl->step_base, &sb, 8, cudaMemcpyHostToDevice));
    // cursors that follow from the step
    e->ce_next = 0;
    while (e->ce_next < e->ce_step.size() && e->ce_step[e->ce_next] < e->step) ++e->ce_next;
    e->ce_group_next = 0;
    while (e->ce_group_next < e->ce_group_step.size() && e->ce_group_step[e->ce_group_next] < e->step) ++e->ce_group_next;
    if (!e->probe_ids.empty()) {
        e->samples_drained = e->step / e->probe_interval;
        const uint32_t s32 = (uint32_t)e->samples_drained;
        CU(cudaMemcpy(&e->d_ctl->sample_base, &s32, 4, cudaMemcpyHostToDevice));
    }
    e->h_spk_n = 0;
    e->log_base_step = e->step;
    e->h_trace.clear();
    // descriptors and exchange words left from steps after the restored one would carry tags that come again
    if (e->d_xchg && e->xp_off)
        CU(cudaMemset(e->d_xchg + kXDescWords + e->xp_off, 0, 8 * xpipe_words((uint32_t)e->n_ranks, (uint32_t)std::max(e->persist_blocks, e->pipe_blocks))));
    if (e->d_pipe_seg) CU(cudaMemset(e->d_pipe_seg, 0, sizeof(uint4) * 3 * (size_t)e->pipe_blocks * kPipeSegCap));
    // replayed inputs handed over before the load are re-indexed from the restored step
    return BMTK_OK;
}

int bmtk_engine_block_profile(bmtk_engine* e, uint64_t cap_blocks, uint64_t* out4, uint64_t* n_blocks) {
    if (!e || !e->finalized || !n_blocks) return fail(BMTK_E_INVALID, "block_profile: engine missing, not finalized, or NULL");
    *n_blocks = e->d_blk_prof ? (uint64_t)e->pipe_blocks : 0;
    if (!e->d_blk_prof || !out4) return BMTK_OK;
    if (cap_blocks < *n_blocks * 5 + 40) return fail(BMTK_E_INVALID, "block_profile: room for %llu blocks, %llu needed",
                                            (unsigned long long)cap_blocks, (unsigned long long)*n_blocks);
    int rc = set_device(e);
    if (rc) return rc;
    CU(cudaStreamSynchronize(e->stream));
    CU(cudaMemcpy(out4, e->d_blk_prof, 32 * (size_t)e->pipe_blocks + 8 * 160 + 128 * (size_t)e->pipe_blocks, cudaMemcpyDeviceToHost));
    CU(cudaMemset(e->d_blk_prof, 0, 32 * (size_t)e->pipe_blocks + 8 * 160 + 128 * (size_t)e->pipe_blocks));
    return BMTK_OK;
}

int bmtk_engine_mark(bmtk_engine* e, int slot) {
    if (!e || slot < 0 || slot >= 8) return fail(BMTK_E_INVALID, "mark: slot must be 0..7");
    int rc = set_device(e);
    if (rc) return rc;
    if (!e->marks[slot]) CU(cudaEventCreate(&e->marks[slot]));
    CU(cudaEventRecord(e->marks[slot], e->stream));
    return BMTK_OK;
}

int bmtk_engine_elapsed_ms(bmtk_engine* e, int from_slot, int to_slot, double* ms) {
    if (!e || !ms || from_slot < 0 || from_slot >= 8 || to_slot < 0 || to_slot >= 8 || !e->marks[from_slot] ||
        !e->marks[to_slot])
        return fail(BMTK_E_INVALID, "elapsed_ms: both slots must have been marked");
    int rc = set_device(e);
    if (rc) return rc;
    CU(cudaEventSynchronize(e->marks[to_slot]));
    float f = 0.f;
    CU(cudaEventElapsedTime(&f, e->marks[from_slot], e->marks[to_slot]));
    *ms = (double)f;
    return BMTK_OK;
}

int bmtk_engine_get_counter(bmtk_engine* e, const char* name, uint64_t* out) {
    if (!e || !name || !out) return fail(BMTK_E_INVALID, "get_counter: NULL argument");
    const std::string k(name);
    if (k == "events") *out = e->events_total;
    else if (k == "spikes") *out = e->spikes_total;
    else if (k == "input_spikes") *out = e->input_spikes_total;
    else if (k == "steps") *out = e->step;
    else if (k == "launches") *out = e->launches;
    else if (k == "window") *out = e->window;
    else if (k == "update_ns") *out = (uint64_t)e->update_ns;
    else if (k == "propagate_ns") *out = (uint64_t)e->prop_ns;
    else if (k == "update_launches") *out = e->update_launches;
    else if (k == "propagate_launches") *out = e->prop_launches;
    else if (k == "spike_capacity") *out = e->send_cap;
    else if (k == "phase_update_ns") *out = (uint64_t)e->phase_update_ns;
    else if (k == "phase_propagate_ns") *out = (uint64_t)e->phase_prop_ns;
    else if (k == "phase_windows") *out = e->phase_windows;
    else if (k == "phase_sync1_ns") *out = (uint64_t)e->phase_sync1_ns;
    else if (k == "phase_sync2_ns") *out = (uint64_t)e->phase_sync2_ns;
    else if (k == "drain_wait_ns") *out = (uint64_t)e->drain_wait_ns;
    else if (k == "drain_sort_ns") *out = (uint64_t)e->drain_sort_ns;
    else if (k == "phase_rows_ns") *out = (uint64_t)e->phase_rows_ns;
    else if (k == "phase_remote_wait_ns") *out = (uint64_t)e->phase_remote_wait_ns;
    else if (k == "phase_remote_rows_ns") *out = (uint64_t)e->phase_remote_rows_ns;
    else if (k == "replays") *out = e->replays;
    else if (k == "log_capacity") *out = e->log_cap;
    else if (k == "event_capacity") *out = e->event_cap;
    else if (k == "persistent_blocks") *out = (uint64_t)e->persist_blocks;
    else if (k == "persistent_resident") *out = e->persist_resident ? 1 : 0;
    else if (k == "pipeline_update_warps") *out = e->pipe_upd_warps;
    else if (k == "pipelined") *out = use_pipelined(e) ? 1 : 0;
    else if (k == "n_pad") *out = e->n_pad;
    else if (k == "n_pad1") *out = e->n_pad1;
    else if (k == "pipeline_trials") *out = e->pipe_trials;
    else if (k == "trials") *out = e->n_trials;
    else return fail(BMTK_E_INVALID, "unknown counter '%s'", name);
    return BMTK_OK;
}

}  // extern "C"
