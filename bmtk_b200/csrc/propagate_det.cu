// Spike-to-synapse propagation, deterministic variant: a sorted segmented reduction.
//
// Per window: (1) the window's spikes are collected as 64-bit keys (emit step, source row) and
// sorted, which makes their order independent of how the update kernel's atomics interleaved;
// (2) row lengths are scanned into event offsets; (3) every event is expanded to
// (ring cell index, weight) in (spike order, row order); (4) a stable radix sort by ring cell
// brings equal cells together without reordering them; (5) one thread per segment sums its
// weights left to right and adds the sum to the ring cell. Every fp32 addition therefore
// happens in one fixed order, whatever the thread scheduling or the number of ranks.
// The radix sorts and the scan are CUB; expansion and reduction are written here.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "propagate_det.cuh"

namespace bmtk {

constexpr int kDetThreads = 128;
constexpr int kDetMaxSeg = 16;

__device__ __forceinline__ uint32_t det_min(uint32_t a, uint32_t b) { return a < b ? a : b; }

// Single block: flattens the window's spike lists into item_keys and publishes the count.
__global__ void det_collect_kernel(const PropArgs a, unsigned long long* keys, uint32_t item_cap) {
    __shared__ uint32_t s_off[kDetMaxSeg + 3];
    __shared__ uint32_t s_in_begin;
    const unsigned long long step_base = a.ctl->step_base;
    if (threadIdx.x == 0) {
        uint32_t tot = 0;
        for (uint32_t r = 0; r < a.n_seg; ++r) {
            s_off[r] = tot;
            tot += det_min(a.gathered[(size_t)r * a.seg_stride], a.seg_cap);
        }
        s_off[a.n_seg] = tot;
        uint32_t n_in = 0;
        s_in_begin = 0;
        if (a.in_ptr) {
            unsigned long long lo = step_base > a.in_ptr_base ? step_base - a.in_ptr_base : 0ull;
            unsigned long long hi = step_base + a.window > a.in_ptr_base ? step_base + a.window - a.in_ptr_base : 0ull;
            const unsigned long long last = a.in_ptr_len - 1;
            if (lo > last) lo = last;
            if (hi > last) hi = last;
            s_in_begin = a.in_ptr[lo];
            n_in = a.in_ptr[hi] - s_in_begin;
        }
        tot += n_in;
        s_off[a.n_seg + 1] = tot;
        tot += a.virt ? det_min(a.virt[0], a.virt_cap) : 0u;
        s_off[a.n_seg + 2] = tot;
        a.ctl->det_items = tot;
    }
    __syncthreads();
    const uint32_t total = det_min(s_off[a.n_seg + 2], item_cap);
    for (uint32_t r = 0; r < a.n_seg; ++r) {
        const uint32_t b = s_off[r], n = s_off[r + 1] - b;
        for (uint32_t i = threadIdx.x; i < n && b + i < total; i += blockDim.x) {
            const uint32_t e = a.gathered[(size_t)r * a.seg_stride + 1 + i];
            keys[b + i] = ((step_base + (e >> kSrcBits)) << 32) | (e & kSrcMask);
        }
    }
    {
        const uint32_t b = s_off[a.n_seg], n = s_off[a.n_seg + 1] - b;
        for (uint32_t i = threadIdx.x; i < n && b + i < total; i += blockDim.x)
            keys[b + i] = ((unsigned long long)a.in_step[s_in_begin + i] << 32) | a.in_src[s_in_begin + i];
    }
    {
        const uint32_t b = s_off[a.n_seg + 1], n = s_off[a.n_seg + 2] - b;
        for (uint32_t i = threadIdx.x; i < n && b + i < total; i += blockDim.x) {
            const uint32_t e = a.virt[1 + i];
            keys[b + i] = ((step_base + (e >> kSrcBits)) << 32) | (e & kSrcMask);
        }
    }
}

__global__ void det_rowlen_kernel(uint32_t n, const unsigned long long* keys, const unsigned long long* rowptr,
                                  uint32_t* len) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const uint32_t src = (uint32_t)keys[i];
        len[i] = (uint32_t)(rowptr[src + 1] - rowptr[src]);
    }
}

// Publishes the event total of the window (last offset + last length).
__global__ void det_total_kernel(uint32_t n, const uint32_t* off, const uint32_t* len, Ctl* ctl) {
    ctl->det_events = n ? off[n - 1] + len[n - 1] : 0u;
}

// One block per spike row: event j of the row goes to position off + j.
__global__ void __launch_bounds__(kDetThreads) det_expand_kernel(uint32_t n, const unsigned long long* keys,
                                                                 const uint32_t* off, const PropArgs a,
                                                                 uint32_t* ev_key, float* ev_val) {
    const uint32_t tb = a.target_bits, tmask = (1u << tb) - 1u;
    for (uint32_t i = blockIdx.x; i < n; i += gridDim.x) {
        const unsigned long long k = keys[i];
        const uint32_t src = (uint32_t)k;
        const uint32_t slot0 = (uint32_t)((k >> 32) % a.ring_slots);
        const unsigned long long b = a.rowptr[src], e = a.rowptr[src + 1];
        const uint32_t o = off[i];
        for (unsigned long long j = threadIdx.x; b + j < e; j += kDetThreads) {
            const uint2 en = a.entries[b + j];
            uint32_t slot = slot0 + (en.x >> (tb + 2));
            if (slot >= a.ring_slots) slot -= a.ring_slots;
            const uint32_t port = (en.x >> tb) & 3u;
            ev_key[o + j] = (slot * kPorts + port) * a.n_pad + (en.x & tmask);
            ev_val[o + j] = __uint_as_float(en.y);
        }
    }
}

// Thread i owns the segment that starts at i (key differs from its left neighbour).
__global__ void det_reduce_kernel(uint32_t n, const uint32_t* key, const float* val, float* ring) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t k = key[i];
    if (i > 0 && key[i - 1] == k) return;
    float sum = val[i];
    for (uint32_t j = i + 1; j < n && key[j] == k; ++j) sum += val[j];
    ring[k] += sum;
}

__global__ void det_window_end_kernel(const PropArgs a, unsigned long long events) {
    a.ctl->n_events += events;
    a.ctl->step_base += a.window;
    if (a.send) a.send[0] = 0u;
    if (a.virt) a.virt[0] = 0u;
}

cudaError_t det_alloc(DetWorkspace& w, uint32_t event_cap, uint32_t item_cap, uint64_t ring_cells) {
    w.event_cap = event_cap;
    w.item_cap = item_cap;
    w.cell_bits = 1;
    while (w.cell_bits < 32 && (ring_cells >> w.cell_bits) != 0) ++w.cell_bits;
    cudaError_t e;
#define DA(p, bytes) if ((e = cudaMalloc(&(p), (bytes))) != cudaSuccess) return e
    DA(w.item_keys, 8ull * item_cap);
    DA(w.item_keys2, 8ull * item_cap);
    DA(w.row_len, 4ull * item_cap);
    DA(w.row_off, 4ull * item_cap);
    DA(w.ev_key, 4ull * event_cap);
    DA(w.ev_key2, 4ull * event_cap);
    DA(w.ev_val, 4ull * event_cap);
    DA(w.ev_val2, 4ull * event_cap);
    size_t t1 = 0, t2 = 0, t3 = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, t1, w.item_keys, w.item_keys2, (int)item_cap);
    cub::DeviceScan::ExclusiveSum(nullptr, t2, w.row_len, w.row_off, (int)item_cap);
    cub::DeviceRadixSort::SortPairs(nullptr, t3, w.ev_key, w.ev_key2, w.ev_val, w.ev_val2, (int)event_cap);
    w.cub_tmp_bytes = t1 > t2 ? t1 : t2;
    if (t3 > w.cub_tmp_bytes) w.cub_tmp_bytes = t3;
    DA(w.cub_tmp, w.cub_tmp_bytes + 16);
#undef DA
    return cudaMallocHost(&w.h_pinned, 16);
}

void det_free(DetWorkspace& w) {
    cudaFree(w.item_keys); cudaFree(w.item_keys2); cudaFree(w.row_len); cudaFree(w.row_off);
    cudaFree(w.ev_key); cudaFree(w.ev_key2); cudaFree(w.ev_val); cudaFree(w.ev_val2); cudaFree(w.cub_tmp);
    if (w.h_pinned) cudaFreeHost(w.h_pinned);
    w = DetWorkspace{};
}

#define DC(x) if ((x) != cudaSuccess) return -1

int propagate_det_window(const PropArgs& a, DetWorkspace& w, cudaStream_t s, uint64_t* launches) {
    det_collect_kernel<<<1, 256, 0, s>>>(a, w.item_keys, w.item_cap);
    DC(cudaGetLastError());
    DC(cudaMemcpyAsync(w.h_pinned, &a.ctl->det_items, 4, cudaMemcpyDeviceToHost, s));
    DC(cudaStreamSynchronize(s));
    *launches += 1;
    const uint32_t n_items = w.h_pinned[0];
    if (n_items > w.item_cap) return -2;
    uint32_t n_events = 0;
    if (n_items) {
        size_t tmp = w.cub_tmp_bytes;
        DC(cub::DeviceRadixSort::SortKeys(w.cub_tmp, tmp, w.item_keys, w.item_keys2, (int)n_items, 0, 64, s));
        det_rowlen_kernel<<<(n_items + 255) / 256, 256, 0, s>>>(n_items, w.item_keys2, a.rowptr, w.row_len);
        DC(cudaGetLastError());
        tmp = w.cub_tmp_bytes;
        DC(cub::DeviceScan::ExclusiveSum(w.cub_tmp, tmp, w.row_len, w.row_off, (int)n_items, s));
        det_total_kernel<<<1, 1, 0, s>>>(n_items, w.row_off, w.row_len, a.ctl);
        DC(cudaGetLastError());
        DC(cudaMemcpyAsync(w.h_pinned + 1, &a.ctl->det_events, 4, cudaMemcpyDeviceToHost, s));
        DC(cudaStreamSynchronize(s));
        n_events = w.h_pinned[1];
        *launches += 4;
        if (n_events > w.event_cap) return -2;
    }
    if (n_events) {
        const uint32_t blocks = n_items < 148u * 8u ? n_items : 148u * 8u;
        det_expand_kernel<<<blocks, kDetThreads, 0, s>>>(n_items, w.item_keys2, w.row_off, a, w.ev_key, w.ev_val);
        DC(cudaGetLastError());
        size_t tmp = w.cub_tmp_bytes;
        DC(cub::DeviceRadixSort::SortPairs(w.cub_tmp, tmp, w.ev_key, w.ev_key2, w.ev_val, w.ev_val2, (int)n_events, 0,
                                           w.cell_bits, s));
        det_reduce_kernel<<<(n_events + 255) / 256, 256, 0, s>>>(n_events, w.ev_key2, w.ev_val2, a.ring);
        DC(cudaGetLastError());
        *launches += 3;
    }
    det_window_end_kernel<<<1, 1, 0, s>>>(a, (unsigned long long)n_events);
    DC(cudaGetLastError());
    *launches += 1;
    return 0;
}

}  // namespace bmtk
