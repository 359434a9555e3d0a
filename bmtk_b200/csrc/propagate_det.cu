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

#include <atomic>
#include <cstdio>
#include <string>

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
        const unsigned long long l = rowptr[src + 1] - rowptr[src];
        len[i] = l > 0xffffffffull ? 0xffffffffu : (uint32_t)l;   // a longer row exceeds every capacity on its own
    }
}

// Publishes the event total of the window. One block; the row lengths are summed in 64 bits and the
// result saturates at 2^32 - 1, so a list whose rows add up to 2^32 events or more (a source may be
// listed many times) can never look small to the capacity check that follows. While the total is
// within a capacity below 2^32, no partial sum of the 32-bit offset scan has wrapped either.
__global__ void det_total_kernel(uint32_t n, const uint32_t* len, Ctl* ctl) {
    __shared__ unsigned long long s_sum[256];
    unsigned long long t = 0ull;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) t += len[i];
    s_sum[threadIdx.x] = t;
    __syncthreads();
    for (uint32_t d = blockDim.x / 2; d > 0; d >>= 1) {
        if (threadIdx.x < d) s_sum[threadIdx.x] += s_sum[threadIdx.x + d];
        __syncthreads();
    }
    if (threadIdx.x == 0) ctl->det_events = s_sum[0] > 0xffffffffull ? 0xffffffffu : (uint32_t)s_sum[0];
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
        det_total_kernel<<<1, 256, 0, s>>>(n_items, w.row_len, a.ctl);
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

// =============================================================================================
// Allocation-free variant of the deterministic delivery.
//
// Some hosts of this library may not allocate device memory at the moment they need a delivery:
// a simulator plugin that runs inside someone else's memory pool (its budget was fixed when the
// pool was carved up), a real-time control loop that must not enter the allocator's locks, or a
// process whose GPU is already filled to the last byte by the network itself. For them the
// scratch of the sorted segmented reduction lives in a fixed array inside the library image.
// Cost: every GPU that loads the library carries the array (about 8.3 MB) until the process exits,
// and one call handles at most kNoAllocMaxSpikes spike rows and kNoAllocMaxEvents synaptic events.
namespace bmtk {

constexpr uint32_t kNoAllocMaxSpikes = 4096;
constexpr uint32_t kNoAllocMaxEvents = 1u << 18;
constexpr size_t kNoAllocCubBytes = 4u << 20;

constexpr size_t na_align(size_t x) { return (x + 255) / 256 * 256; }
constexpr size_t kNaCtl = 0;
constexpr size_t kNaInPtr = kNaCtl + na_align(sizeof(Ctl));
constexpr size_t kNaItemKeys = kNaInPtr + na_align(2 * sizeof(uint32_t));
constexpr size_t kNaItemKeys2 = kNaItemKeys + na_align(8ull * kNoAllocMaxSpikes);
constexpr size_t kNaRowLen = kNaItemKeys2 + na_align(8ull * kNoAllocMaxSpikes);
constexpr size_t kNaRowOff = kNaRowLen + na_align(4ull * kNoAllocMaxSpikes);
constexpr size_t kNaEvKey = kNaRowOff + na_align(4ull * kNoAllocMaxSpikes);
constexpr size_t kNaEvKey2 = kNaEvKey + na_align(4ull * kNoAllocMaxEvents);
constexpr size_t kNaEvVal = kNaEvKey2 + na_align(4ull * kNoAllocMaxEvents);
constexpr size_t kNaEvVal2 = kNaEvVal + na_align(4ull * kNoAllocMaxEvents);
constexpr size_t kNaCub = kNaEvVal2 + na_align(4ull * kNoAllocMaxEvents);
constexpr size_t kNoAllocBytes = kNaCub + kNoAllocCubBytes;

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress: it is not
// a device address and must never be handed to a kernel as a pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNaMaxDevices = 64;
// device address of the array, per device; atomic so that first calls racing from two host threads are defined
// (both store the same value)
static std::atomic<unsigned char*> g_noalloc_addr[kNaMaxDevices];

extern thread_local std::string g_last_error;

static int na_fail(int code, const char* msg, cudaError_t ce = cudaSuccess) {
    char buf[512];
    if (ce != cudaSuccess) snprintf(buf, sizeof(buf), "propagate_spikes_noalloc: %s: %s", msg, cudaGetErrorString(ce));
    else snprintf(buf, sizeof(buf), "propagate_spikes_noalloc: %s", msg);
    g_last_error = buf;
    return code;
}

// Zeroes the control block (it keeps the previous call's counters) and writes the [0, n) slice
// table through which the collect kernel finds the caller's spike list.
__global__ void noalloc_setup_kernel(Ctl* ctl, uint32_t* in_ptr, uint32_t n_spikes) {
    Ctl z{};
    *ctl = z;
    in_ptr[0] = 0u;
    in_ptr[1] = n_spikes;
}

}  // namespace bmtk

extern "C" __attribute__((visibility("default")))
int bmtk_propagate_spikes_noalloc(const uint64_t* d_rowptr, const void* d_entries, uint32_t target_bits,
                                  uint32_t n_spikes, const uint32_t* d_spike_src, const uint32_t* d_spike_step,
                                  float* d_ring, uint32_t ring_slots, uint32_t n_pad, void* stream) {
    using namespace bmtk;
    if (!d_rowptr || !d_entries || !d_ring) return na_fail(BMTK_E_INVALID, "NULL device pointer");
    if (n_spikes && (!d_spike_src || !d_spike_step)) return na_fail(BMTK_E_INVALID, "NULL spike list");
    if (ring_slots < 1 || n_pad < 1 || target_bits < 1 || target_bits > 29)
        return na_fail(BMTK_E_INVALID, "bad ring geometry");
    if (n_spikes > kNoAllocMaxSpikes) {
        char m[160];
        snprintf(m, sizeof(m), "%u spikes in one call, the built-in scratch holds at most %u "
                 "(split the list or use bmtk_propagate_spikes)", n_spikes, kNoAllocMaxSpikes);
        return na_fail(BMTK_E_INVALID, m);
    }
    const uint64_t cells = (uint64_t)ring_slots * kPorts * n_pad;
    if (cells >= (1ull << 32)) return na_fail(BMTK_E_UNSUPPORTED, "ring has 2^32 cells or more");
    if (n_spikes == 0) return BMTK_OK;

    // Once per device, with that device current: ask the runtime where the array lives there.
    int dev = -1;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return na_fail(BMTK_E_CUDA, "cudaGetDevice", ce);
    if (dev < 0 || dev >= kNaMaxDevices) return na_fail(BMTK_E_UNSUPPORTED, "device ordinal beyond 63");
    unsigned char* base = g_noalloc_addr[dev].load(std::memory_order_acquire);
    if (!base) {
        ce = cudaGetSymbolAddress((void**)&base, g_noalloc_scratch);
        if (ce != cudaSuccess || !base) return na_fail(BMTK_E_CUDA, "cudaGetSymbolAddress(scratch)", ce);
        g_noalloc_addr[dev].store(base, std::memory_order_release);
    }
    cudaStream_t st = (cudaStream_t)stream;

    Ctl* ctl = reinterpret_cast<Ctl*>(base + kNaCtl);
    uint32_t* in_ptr = reinterpret_cast<uint32_t*>(base + kNaInPtr);
    unsigned long long* item_keys = reinterpret_cast<unsigned long long*>(base + kNaItemKeys);
    unsigned long long* item_keys2 = reinterpret_cast<unsigned long long*>(base + kNaItemKeys2);
    uint32_t* row_len = reinterpret_cast<uint32_t*>(base + kNaRowLen);
    uint32_t* row_off = reinterpret_cast<uint32_t*>(base + kNaRowOff);
    uint32_t* ev_key = reinterpret_cast<uint32_t*>(base + kNaEvKey);
    uint32_t* ev_key2 = reinterpret_cast<uint32_t*>(base + kNaEvKey2);
    float* ev_val = reinterpret_cast<float*>(base + kNaEvVal);
    float* ev_val2 = reinterpret_cast<float*>(base + kNaEvVal2);
    void* cub_tmp = base + kNaCub;

    int cell_bits = 1;
    while (cell_bits < 32 && (cells >> cell_bits) != 0) ++cell_bits;

    // CUB is handed its temporary storage; ask how much each call wants and refuse if the
    // reserved region were too small (sizes are fixed by the maxima above, so this never trips).
    size_t t1 = 0, t2 = 0, t3 = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, t1, item_keys, item_keys2, (int)kNoAllocMaxSpikes, 0, 64, st);
    cub::DeviceScan::ExclusiveSum(nullptr, t2, row_len, row_off, (int)kNoAllocMaxSpikes, st);
    cub::DeviceRadixSort::SortPairs(nullptr, t3, ev_key, ev_key2, ev_val, ev_val2, (int)kNoAllocMaxEvents, 0, cell_bits, st);
    if (t1 > kNoAllocCubBytes || t2 > kNoAllocCubBytes || t3 > kNoAllocCubBytes)
        return na_fail(BMTK_E_UNSUPPORTED, "sort workspace exceeds the built-in scratch");

    noalloc_setup_kernel<<<1, 1, 0, st>>>(ctl, in_ptr, n_spikes);
    if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "set-up launch", ce);

    PropArgs a{};
    a.rowptr = (const unsigned long long*)d_rowptr;
    a.entries = (const uint2*)d_entries;
    a.target_bits = target_bits;
    a.ring = d_ring;
    a.ring_slots = ring_slots;
    a.n_pad = n_pad;
    a.ctl = ctl;
    a.n_seg = 0;
    a.in_ptr = in_ptr;
    a.in_ptr_base = 0;
    a.in_ptr_len = 2;
    a.in_step = d_spike_step;
    a.in_src = d_spike_src;
    a.window = 1;

    det_collect_kernel<<<1, 256, 0, st>>>(a, item_keys, kNoAllocMaxSpikes);
    if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "collect launch", ce);
    size_t tmp = kNoAllocCubBytes;
    if ((ce = cub::DeviceRadixSort::SortKeys(cub_tmp, tmp, item_keys, item_keys2, (int)n_spikes, 0, 64, st)) != cudaSuccess)
        return na_fail(BMTK_E_CUDA, "spike sort", ce);
    det_rowlen_kernel<<<(n_spikes + 255) / 256, 256, 0, st>>>(n_spikes, item_keys2, a.rowptr, row_len);
    if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "row-length launch", ce);
    tmp = kNoAllocCubBytes;
    if ((ce = cub::DeviceScan::ExclusiveSum(cub_tmp, tmp, row_len, row_off, (int)n_spikes, st)) != cudaSuccess)
        return na_fail(BMTK_E_CUDA, "offset scan", ce);
    det_total_kernel<<<1, 256, 0, st>>>(n_spikes, row_len, ctl);
    if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "total launch", ce);
    uint32_t n_events = 0;
    if ((ce = cudaMemcpyAsync(&n_events, &ctl->det_events, 4, cudaMemcpyDeviceToHost, st)) != cudaSuccess)
        return na_fail(BMTK_E_CUDA, "event count read-back", ce);
    if ((ce = cudaStreamSynchronize(st)) != cudaSuccess) return na_fail(BMTK_E_CUDA, "synchronize", ce);
    if (n_events > kNoAllocMaxEvents) {
        char m[200];
        snprintf(m, sizeof(m), "%u synaptic events in one call, the built-in scratch holds at most %u; "
                 "nothing was delivered (split the spike list or use bmtk_propagate_spikes)", n_events, kNoAllocMaxEvents);
        return na_fail(BMTK_E_OVERFLOW, m);
    }
    if (n_events) {
        const uint32_t blocks = n_spikes < 148u * 8u ? n_spikes : 148u * 8u;
        det_expand_kernel<<<blocks, kDetThreads, 0, st>>>(n_spikes, item_keys2, row_off, a, ev_key, ev_val);
        if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "expand launch", ce);
        tmp = kNoAllocCubBytes;
        if ((ce = cub::DeviceRadixSort::SortPairs(cub_tmp, tmp, ev_key, ev_key2, ev_val, ev_val2, (int)n_events, 0,
                                                  cell_bits, st)) != cudaSuccess)
            return na_fail(BMTK_E_CUDA, "event sort", ce);
        det_reduce_kernel<<<(n_events + 255) / 256, 256, 0, st>>>(n_events, ev_key2, ev_val2, d_ring);
        if ((ce = cudaGetLastError()) != cudaSuccess) return na_fail(BMTK_E_CUDA, "reduce launch", ce);
    }
    if ((ce = cudaStreamSynchronize(st)) != cudaSuccess) return na_fail(BMTK_E_CUDA, "synchronize", ce);
    return BMTK_OK;
}
