// Device-side sampler of a distance-dependent point-neuron network: the synthetic stand-in for bmtk.builder on
// this path (the reference builds such networks with per-pair Python connection rules,
// examples/point_450glifs/build_network.py; bmtk/builder/network_adaptors/dm_network.py:103-121 writes them).
//
// For every target neuron t a fixed-rate number of candidate synapses is drawn; candidate k of target t owns the
// Philox4x32-10 counters (t, k, 0, 0) and (t, k, 1, 0) under the key `seed`, so the network does not depend on how
// the work is spread over threads, blocks or GPUs. A candidate picks the class of its source (excitatory /
// inhibitory), a Gaussian displacement with the (class, target type) sigma from a 4096-quantile table, and lands
// in a cell of a square grid over the disk; a cell that holds c neurons of the class keeps the candidate with
// probability c / c_max (so that every neuron is hit in proportion to the kernel at its cell) and hands it to one
// of its neurons uniformly. Weight = base(source type, target type) x a lognormal factor from a second table,
// negative for inhibitory sources; delay uniform on the dt grid; receptor port by class pair.
//
// All arithmetic is integer work or single IEEE-754 operations in a fixed order (explicit fused multiply-adds, no
// transcendental function: the two tables are made by the host once), so a CPU restatement reproduces the edge
// list bit for bit. Pass 1 counts the accepted candidates per target, a CUB scan turns counts into offsets, pass 2
// writes the edges in (target, candidate) order.
#include <cub/device/device_scan.cuh>

#include <string>
#include <vector>

#include "common.cuh"
#include "philox.cuh"

namespace bmtk {

struct GenDev {
    bmtk_gen_spec s;              // host pointers inside are replaced by the device copies below
    const uint16_t* type_index;
    const uint8_t* type_is_inh;
    const float *x, *y, *sigma, *w_base, *q_exc, *q_inh, *lambda, *gauss, *lognorm;
    const uint32_t *cell_start[2], *cell_count[2], *cell_ids[2];
    float cmax[2];
};

struct Candidate {
    uint32_t src;
    float weight;
    uint16_t delay;
    uint8_t port;
    bool ok;
};

__host__ __device__ __forceinline__ float u24(uint32_t r) { return (float)(r >> 8) * 5.9604644775390625e-08f; }   // [0, 1), exact

__device__ __forceinline__ uint32_t candidates_of(const GenDev& g, uint32_t t) {
    const float lam = g.lambda[g.type_index[t]];
    const uint32_t base = (uint32_t)lam;
    const uint4 r = philox4x32_10(t, 0xffffffffu, 2u, 0u, (uint32_t)g.s.seed, (uint32_t)(g.s.seed >> 32));
    return base + (u24(r.x) < lam - (float)base ? 1u : 0u);
}

__device__ __forceinline__ Candidate draw(const GenDev& g, uint32_t t, uint32_t k) {
    Candidate c;
    c.ok = false;
    const uint32_t k0 = (uint32_t)g.s.seed, k1 = (uint32_t)(g.s.seed >> 32);
    const uint4 a = philox4x32_10(t, k, 0u, 0u, k0, k1);
    const uint4 b = philox4x32_10(t, k, 1u, 0u, k0, k1);
    const uint32_t tt = g.type_index[t];
    const float qe = g.q_exc[tt], qi = g.q_inh[tt];
    const uint32_t sc = __fmul_rn(u24(a.x), __fadd_rn(qe, qi)) >= qe ? 1u : 0u;
    const float sg = g.sigma[sc * g.s.n_types + tt];
    const float px = __fmaf_rn(g.gauss[a.y >> 20], sg, g.x[t]);
    const float py = __fmaf_rn(g.gauss[a.z >> 20], sg, g.y[t]);
    const float R = g.s.radius;
    if (!(__fmaf_rn(px, px, __fmul_rn(py, py)) < __fmul_rn(R, R))) return c;
    const int cx = (int)floorf(__fmul_rn(__fadd_rn(px, R), g.s.inv_cell));
    const int cy = (int)floorf(__fmul_rn(__fadd_rn(py, R), g.s.inv_cell));
    if (cx < 0 || cy < 0 || cx >= (int)g.s.grid || cy >= (int)g.s.grid) return c;
    const uint32_t key = (uint32_t)cx * g.s.grid + (uint32_t)cy;
    const uint32_t cn = g.cell_count[sc][key];
    if (!(__fmul_rn(u24(a.w), g.cmax[sc]) < (float)cn)) return c;
    uint32_t pick = (uint32_t)__fmul_rn(u24(b.x), (float)cn);
    if (pick >= cn) pick = cn - 1u;
    const uint32_t s = g.cell_ids[sc][g.cell_start[sc][key] + pick];
    if (s == t) return c;
    const uint32_t st = g.type_index[s];
    float w = __fmul_rn(g.w_base[st * g.s.n_types + tt], g.lognorm[b.y >> 20]);
    const bool s_inh = g.type_is_inh[st] != 0, t_inh = g.type_is_inh[tt] != 0;
    if (s_inh) w = __fmul_rn(w, -g.s.inh_scale);
    const float d_ms = __fmaf_rn(u24(b.z), __fsub_rn(g.s.delay_max_ms, g.s.delay_min_ms), g.s.delay_min_ms);
    const float d_steps = rintf(__fdiv_rn(d_ms, g.s.dt));
    c.src = s;
    c.weight = w;
    c.delay = (uint16_t)(d_steps < 1.f ? 1.f : d_steps);
    c.port = (uint8_t)((s_inh ? 1u : 0u) + (t_inh ? 2u : 0u));
    c.ok = true;
    return c;
}

// One warp per target: lanes stride over the target's candidates.
__global__ void gen_count_kernel(const GenDev g, uint32_t lo, uint32_t hi, unsigned long long* counts) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t t = lo + warp; t < hi; t += n_warps) {
        const uint32_t K = candidates_of(g, t);
        uint32_t n = 0;
        for (uint32_t k0 = 0; k0 < K; k0 += 32u) {
            const bool ok = k0 + lane < K && draw(g, t, k0 + lane).ok;
            n += __popc(__ballot_sync(0xffffffffu, ok));
        }
        if (lane == 0) counts[t - lo] = n;
    }
}

__global__ void gen_fill_kernel(const GenDev g, uint32_t lo, uint32_t hi, const unsigned long long* offsets, uint32_t* src,
                                uint32_t* trg, float* weight, uint16_t* delay, uint8_t* port) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t t = lo + warp; t < hi; t += n_warps) {
        const uint32_t K = candidates_of(g, t);
        unsigned long long o = offsets[t - lo];
        for (uint32_t k0 = 0; k0 < K; k0 += 32u) {
            Candidate c;
            c.ok = false;
            if (k0 + lane < K) c = draw(g, t, k0 + lane);
            const uint32_t m = __ballot_sync(0xffffffffu, c.ok);
            if (c.ok) {
                const unsigned long long p = o + __popc(m & ((1u << lane) - 1u));
                src[p] = c.src;
                trg[p] = t;
                weight[p] = c.weight;
                delay[p] = c.delay;
                port[p] = c.port;
            }
            o += __popc(m);
        }
    }
}

extern thread_local std::string g_last_error;

static int gen_fail(int code, const char* msg, cudaError_t ce = cudaSuccess) {
    g_last_error = std::string("generate_distance_edges: ") + msg + (ce != cudaSuccess ? std::string(": ") + cudaGetErrorString(ce) : "");
    return code;
}

}  // namespace bmtk

using namespace bmtk;

extern "C" __attribute__((visibility("default")))
int bmtk_generate_distance_edges(const bmtk_gen_spec* spec, int device, uint64_t cap, uint32_t* src, uint32_t* trg, float* weight,
                                 uint16_t* delay_steps, uint8_t* port, uint64_t* n_edges) {
    if (!spec || !n_edges) return gen_fail(BMTK_E_INVALID, "NULL argument");
    const bmtk_gen_spec& s = *spec;
    if (s.n_neurons < 1 || s.n_types < 1 || s.hi > s.n_neurons || s.lo > s.hi || s.grid < 1 || !(s.dt > 0) || !(s.inv_cell > 0))
        return gen_fail(BMTK_E_INVALID, "bad specification");
    if (!s.type_index || !s.type_is_inh || !s.x || !s.y || !s.sigma || !s.w_base || !s.q_exc || !s.q_inh || !s.lambda ||
        !s.gauss_table || !s.lognorm_table)
        return gen_fail(BMTK_E_INVALID, "NULL table in the specification");
    for (int c = 0; c < 2; ++c)
        if (!s.cell_start[c] || !s.cell_count[c] || (s.class_size[c] && !s.cell_ids[c]))
            return gen_fail(BMTK_E_INVALID, "NULL grid table in the specification");
    cudaError_t ce = cudaSetDevice(device);
    if (ce != cudaSuccess) return gen_fail(BMTK_E_CUDA, "cudaSetDevice", ce);
    std::vector<void*> owned;
    auto up = [&](const void* h, size_t bytes) -> void* {
        void* d = nullptr;
        if (cudaMalloc(&d, bytes ? bytes : 4) != cudaSuccess) return nullptr;
        owned.push_back(d);
        if (h && bytes && cudaMemcpy(d, h, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
        return d;
    };
    auto cleanup = [&]() { for (void* p : owned) cudaFree(p); };
    GenDev g{};
    g.s = s;
    const size_t n = s.n_neurons, nt = s.n_types, cells = (size_t)s.grid * s.grid;
    g.type_index = (const uint16_t*)up(s.type_index, 2 * n);
    g.type_is_inh = (const uint8_t*)up(s.type_is_inh, nt);
    g.x = (const float*)up(s.x, 4 * n);
    g.y = (const float*)up(s.y, 4 * n);
    g.sigma = (const float*)up(s.sigma, 4 * 2 * nt);
    g.w_base = (const float*)up(s.w_base, 4 * nt * nt);
    g.q_exc = (const float*)up(s.q_exc, 4 * nt);
    g.q_inh = (const float*)up(s.q_inh, 4 * nt);
    g.lambda = (const float*)up(s.lambda, 4 * nt);
    g.gauss = (const float*)up(s.gauss_table, 4 * 4096);
    g.lognorm = (const float*)up(s.lognorm_table, 4 * 4096);
    bool ok = g.type_index && g.type_is_inh && g.x && g.y && g.sigma && g.w_base && g.q_exc && g.q_inh && g.lambda && g.gauss && g.lognorm;
    for (int c = 0; c < 2 && ok; ++c) {
        g.cell_start[c] = (const uint32_t*)up(s.cell_start[c], 4 * cells);
        g.cell_count[c] = (const uint32_t*)up(s.cell_count[c], 4 * cells);
        g.cell_ids[c] = (const uint32_t*)up(s.cell_ids[c], 4 * (size_t)s.class_size[c]);
        g.cmax[c] = s.cell_max[c];
        ok = g.cell_start[c] && g.cell_count[c] && g.cell_ids[c];
    }
    if (!ok) { cleanup(); return gen_fail(BMTK_E_CUDA, "device allocation or upload failed", cudaGetLastError()); }
    const uint32_t n_t = s.hi - s.lo;
    unsigned long long *d_cnt = nullptr, *d_off = nullptr;
    void* d_tmp = nullptr;
    size_t tmp_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, d_cnt, d_off, (int)n_t + 1);
    d_cnt = (unsigned long long*)up(nullptr, 8 * ((size_t)n_t + 1));
    d_off = (unsigned long long*)up(nullptr, 8 * ((size_t)n_t + 1));
    d_tmp = up(nullptr, tmp_bytes);
    if (!d_cnt || !d_off || !d_tmp) { cleanup(); return gen_fail(BMTK_E_CUDA, "device allocation failed", cudaGetLastError()); }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int blocks = sms * 8, threads = 256;
    cudaMemset(d_cnt, 0, 8 * ((size_t)n_t + 1));
    if (n_t) gen_count_kernel<<<blocks, threads>>>(g, s.lo, s.hi, d_cnt);
    ce = cudaGetLastError();
    if (ce == cudaSuccess) ce = cub::DeviceScan::ExclusiveSum(d_tmp, tmp_bytes, d_cnt, d_off, (int)n_t + 1);
    unsigned long long total = 0;
    if (ce == cudaSuccess) ce = cudaMemcpy(&total, d_off + n_t, 8, cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) { cleanup(); return gen_fail(BMTK_E_CUDA, "counting pass", ce); }
    *n_edges = total;
    if (cap == 0 && !src) { cleanup(); return BMTK_OK; }     // size query
    if (cap < total) { cleanup(); return gen_fail(BMTK_E_INVALID, "capacity below the number of edges (call with cap = 0 first)"); }
    if (total && (!src || !trg || !weight || !delay_steps || !port)) { cleanup(); return gen_fail(BMTK_E_INVALID, "NULL output array"); }
    uint32_t* d_src = (uint32_t*)up(nullptr, 4 * (size_t)total);
    uint32_t* d_trg = (uint32_t*)up(nullptr, 4 * (size_t)total);
    float* d_w = (float*)up(nullptr, 4 * (size_t)total);
    uint16_t* d_d = (uint16_t*)up(nullptr, 2 * (size_t)total);
    uint8_t* d_p = (uint8_t*)up(nullptr, (size_t)total);
    if (!d_src || !d_trg || !d_w || !d_d || !d_p) { cleanup(); return gen_fail(BMTK_E_CUDA, "device allocation for the edges failed", cudaGetLastError()); }
    if (total) gen_fill_kernel<<<blocks, threads>>>(g, s.lo, s.hi, d_off, d_src, d_trg, d_w, d_d, d_p);
    ce = cudaGetLastError();
    if (ce == cudaSuccess && total) {
        ce = cudaMemcpy(src, d_src, 4 * (size_t)total, cudaMemcpyDeviceToHost);
        if (ce == cudaSuccess) ce = cudaMemcpy(trg, d_trg, 4 * (size_t)total, cudaMemcpyDeviceToHost);
        if (ce == cudaSuccess) ce = cudaMemcpy(weight, d_w, 4 * (size_t)total, cudaMemcpyDeviceToHost);
        if (ce == cudaSuccess) ce = cudaMemcpy(delay_steps, d_d, 2 * (size_t)total, cudaMemcpyDeviceToHost);
        if (ce == cudaSuccess) ce = cudaMemcpy(port, d_p, (size_t)total, cudaMemcpyDeviceToHost);
    }
    cleanup();
    if (ce != cudaSuccess) return gen_fail(BMTK_E_CUDA, "fill pass", ce);
    return BMTK_OK;
}
