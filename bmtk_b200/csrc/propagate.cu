// Spike-to-synapse propagation over the delay-bucketed CSR (throughput variant: atomics).
//
// One launch per exchange window. Work items are the spikes of the window: the gathered
// recurrent lists of every rank, the replayed virtual spikes whose emitting step falls in the
// window, and the on-line Poisson spikes. A block takes items blockIdx.x, blockIdx.x + gridDim.x,
// ...; it first stages (row begin, row end, ring slot) of up to kStage of its items in shared
// memory with one thread per item — so the dependent chain spike entry -> row pointers is paid
// once per block, not once per row — then streams each row with all threads: consecutive
// threads read consecutive 8-byte {packed target|port|delay, weight} entries (256 B per warp
// per request, four requests in flight per thread) and issue one fire-and-forget fp32 reduction
// into ring[(emit step + delay) mod slots][port][target].
// Algorithmic traffic: 8 B of CSR payload + 4 B read + 4 B write of the ring cell = 16 B per
// synaptic event. Replaces NEST's event delivery inside nest.Simulate
// (bmtk/simulator/pointnet/pointsimulator.py:166; connections from pointnetwork.py:229-248).
#include "common.cuh"

namespace bmtk {

constexpr int kPropThreads = 128;
constexpr int kStage = 32;
constexpr int kMaxSeg = 16;

struct Item {
    unsigned long long begin, end;
    uint32_t slot0;
    uint32_t cell0;   // first cell of the spike's trial inside a ring plane
};

// Resolves work item `idx` (0 <= idx < total) to (source row, emitting step).
struct ItemMap {
    uint32_t n_rec[kMaxSeg];
    uint32_t n_in, in_begin, n_virt;
    uint32_t total;
};

__device__ __forceinline__ uint32_t clamp_count(uint32_t c, uint32_t cap) { return c < cap ? c : cap; }

__device__ __forceinline__ void build_map(const PropArgs& a, unsigned long long step_base, ItemMap& m) {
    uint32_t tot = 0;
    for (uint32_t r = 0; r < a.n_seg; ++r) {
        m.n_rec[r] = clamp_count(a.gathered[(size_t)r * a.seg_stride], a.seg_cap);
        tot += m.n_rec[r];
    }
    m.n_in = 0;
    m.in_begin = 0;
    if (a.in_ptr) {
        unsigned long long lo = step_base > a.in_ptr_base ? step_base - a.in_ptr_base : 0ull;
        unsigned long long hi = step_base + a.window > a.in_ptr_base ? step_base + a.window - a.in_ptr_base : 0ull;
        const unsigned long long last = a.in_ptr_len - 1;
        if (lo > last) lo = last;
        if (hi > last) hi = last;
        m.in_begin = a.in_ptr[lo];
        m.n_in = a.in_ptr[hi] - m.in_begin;
        tot += m.n_in;
    }
    m.n_virt = a.virt ? clamp_count(a.virt[0], a.virt_cap) : 0u;
    tot += m.n_virt;
    m.total = tot;
}

__device__ __forceinline__ void resolve(const PropArgs& a, const ItemMap& m, unsigned long long step_base,
                                        uint32_t idx, uint32_t& src, unsigned long long& step) {
    for (uint32_t r = 0; r < a.n_seg; ++r) {
        if (idx < m.n_rec[r]) {
            const uint32_t e = a.gathered[(size_t)r * a.seg_stride + 1 + idx];
            src = e & kSrcMask;
            step = step_base + (e >> kSrcBits);
            return;
        }
        idx -= m.n_rec[r];
    }
    if (idx < m.n_in) {
        src = a.in_src[m.in_begin + idx];
        step = a.in_step[m.in_begin + idx];
        return;
    }
    idx -= m.n_in;
    const uint32_t e = a.virt[1 + idx];
    src = e & kSrcMask;
    step = step_base + (e >> kSrcBits);
}

__global__ void __launch_bounds__(kPropThreads) propagate_atomic_kernel(const PropArgs a) {
    __shared__ Item s_items[kStage];
    __shared__ ItemMap s_map;
    __shared__ unsigned long long s_events;
    const unsigned long long step_base = a.ctl->step_base;
    if (threadIdx.x == 0) {
        build_map(a, step_base, s_map);
        s_events = 0ull;
    }
    __syncthreads();
    const uint32_t total = s_map.total;
    const uint32_t tb = a.target_bits;
    const uint32_t tmask = (1u << tb) - 1u;
    const size_t plane = (size_t)a.n_pad;

    for (uint32_t first = blockIdx.x; first < total; first += gridDim.x * kStage) {
        // stage up to kStage items of this block
        if (threadIdx.x < kStage) {
            const uint32_t idx = first + threadIdx.x * gridDim.x;
            Item it = {0ull, 0ull, 0u, 0u};
            if (idx < total) {
                uint32_t src, row, trial;
                unsigned long long step;
                resolve(a, s_map, step_base, idx, src, step);
                split_source(a.ids, src, row, trial);
                it.begin = a.rowptr[row];
                it.end = a.rowptr[row + 1];
                it.slot0 = (uint32_t)(step % a.ring_slots);
                it.cell0 = trial * a.n_pad1;
            }
            s_items[threadIdx.x] = it;
        }
        __syncthreads();
        unsigned long long my_events = 0ull;
#pragma unroll 1
        for (int q = 0; q < kStage; ++q) {
            const Item it = s_items[q];
            if (it.end == it.begin) {
                if (first + (uint32_t)q * gridDim.x >= total) break;
                continue;
            }
            if (threadIdx.x == 0) my_events += it.end - it.begin;
            float* ring0 = a.ring + it.cell0;
            unsigned long long k = it.begin + threadIdx.x;
            // four independent loads in flight per thread
            for (; k + 3ull * kPropThreads < it.end; k += 4ull * kPropThreads) {
                uint2 e[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) e[u] = __ldg(&a.entries[k + (unsigned long long)u * kPropThreads]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint32_t slot = it.slot0 + (e[u].x >> (tb + 2));
                    if (slot >= a.ring_slots) slot -= a.ring_slots;
                    const uint32_t port = (e[u].x >> tb) & 3u;
                    atomicAdd(ring0 + ((size_t)slot * kPorts + port) * plane + (e[u].x & tmask),
                              __uint_as_float(e[u].y));
                }
            }
            for (; k < it.end; k += kPropThreads) {
                const uint2 e = __ldg(&a.entries[k]);
                uint32_t slot = it.slot0 + (e.x >> (tb + 2));
                if (slot >= a.ring_slots) slot -= a.ring_slots;
                const uint32_t port = (e.x >> tb) & 3u;
                atomicAdd(ring0 + ((size_t)slot * kPorts + port) * plane + (e.x & tmask), __uint_as_float(e.y));
            }
        }
        if (threadIdx.x == 0) s_events += my_events;
        __syncthreads();
    }

    // ---- window end: the last block to finish advances the clock and clears the lists
    if (threadIdx.x == 0) {
        if (s_events) atomicAdd(&a.ctl->n_events, s_events);
        __threadfence();
        const uint32_t t = atomicAdd(&a.ctl->ticket, 1u);
        if (t == gridDim.x - 1) {
            a.ctl->ticket = 0u;
            a.ctl->step_base = step_base + a.window;
            if (a.send) a.send[0] = 0u;
            if (a.virt) a.virt[0] = 0u;
            __threadfence();
        }
    }
}

// Ceiling probe for the delivery kernels: `n_ops` fp32 reductions into pseudo-random cells of a
// buffer of `n_cells` floats, nothing else (the address comes from a multiplicative hash of the
// thread's running index, no loads). What this sustains is the most any delivery scheme that ends
// in one scattered reduction per synaptic event can reach on the device.
__global__ void scatter_red_probe_kernel(float* cells, uint32_t n_cells, unsigned long long n_ops) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_ops; i += stride) {
        const uint32_t h = (uint32_t)((i * 0x9E3779B97F4A7C15ull) >> 32);
        atomicAdd(cells + (uint32_t)(((unsigned long long)h * n_cells) >> 32), 1.0f);
    }
}

cudaError_t launch_scatter_red_probe(float* cells, uint32_t n_cells, unsigned long long n_ops, cudaStream_t s) {
    scatter_red_probe_kernel<<<148 * 8, 256, 0, s>>>(cells, n_cells, n_ops);
    return cudaGetLastError();
}

cudaError_t launch_propagate_atomic(const PropArgs& a, cudaStream_t s) {
    if (a.n_seg > kMaxSeg) return cudaErrorInvalidValue;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    static int cached_sms = 0;
    if (!cached_sms) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
        cached_sms = sms;
    }
    // a multiple of the SM count; 8 resident blocks of 128 threads per SM
    const int blocks = cached_sms * 8;
    propagate_atomic_kernel<<<blocks, kPropThreads, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace bmtk
