// Device build of the delay-bucketed CSR from an edge list.
//
// Each edge becomes a 64-bit key  source << 32 | delay << (tb+2) | port << tb | local target
// (tb = bits needed for the local target index) with its fp32 weight as the value. One stable
// radix sort (CUB) orders the edges by source row and, inside a row, by delay bucket, then
// port, then target; equal keys keep their order in the edge list. The low word of the sorted
// key is the CSR entry itself, so the build is sort + one pass that interleaves
// {packed, weight} and one pass that writes the row pointers. The result is bit-identical to
// a host np.lexsort((target, port, delay, source)) construction.
// Replaces the connection tables nest.Connect fills (bmtk/simulator/pointnet/pointnetwork.py:229-248).
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "csr_build.cuh"

namespace bmtk {

__global__ void make_keys_kernel(uint64_t n, const uint32_t* src, const uint32_t* trg, const uint16_t* delay,
                                 const uint8_t* port, uint32_t lo, uint32_t tb, unsigned long long* keys) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint32_t packed = ((uint32_t)delay[i] << (tb + 2)) | ((uint32_t)port[i] << tb) | (trg[i] - lo);
        keys[i] = ((unsigned long long)src[i] << 32) | packed;
    }
}

__global__ void emit_csr_kernel(uint64_t n, uint64_t n_rows, const unsigned long long* keys, const float* w,
                                uint2* entries, unsigned long long* rowptr) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long k = keys[i];
        entries[i] = make_uint2((uint32_t)k, __float_as_uint(w[i]));
        const uint64_t row = k >> 32;
        // rows (prev, row] start at i; row 0.. for the first edge
        const uint64_t prev = i == 0 ? (uint64_t)-1 : (uint64_t)(keys[i - 1] >> 32);
        if (i == 0 || prev != row) {
            for (uint64_t r = (i == 0 ? 0 : prev + 1); r <= row; ++r) rowptr[r] = i;
        }
        if (i == n - 1) {
            for (uint64_t r = row + 1; r <= n_rows; ++r) rowptr[r] = n;
        }
    }
}

__global__ void fill_u64_kernel(unsigned long long* p, uint64_t n, unsigned long long v) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

// spike log: key = (stamp - stamp_base) << id_bits | id, so that the sort runs over the bits in use only
__global__ void pack_log_kernel(uint32_t n, const uint32_t* stamp, const uint32_t* id, uint32_t stamp_base, uint32_t id_bits,
                                unsigned long long* keys) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) keys[i] = ((unsigned long long)(stamp[i] - stamp_base) << id_bits) | id[i];
}

// The same for a log kept in per-block segments of seg_cap entries with counts seg_cnt[n_seg]: thread
// block b packs segment b behind the segments before it (every block adds up the counts before its own).
__global__ void pack_log_segments_kernel(uint32_t n_seg, uint32_t seg_cap, const uint32_t* seg_cnt, const uint32_t* stamp,
                                         const uint32_t* id, uint32_t stamp_base, uint32_t id_bits, unsigned long long* keys) {
    __shared__ uint32_t s_off;
    if (threadIdx.x == 0) {
        uint32_t off = 0;
        for (uint32_t b = 0; b < blockIdx.x; ++b) off += seg_cnt[b];
        s_off = off;
    }
    __syncthreads();
    const uint32_t n = seg_cnt[blockIdx.x], off = s_off;
    const size_t base = (size_t)blockIdx.x * seg_cap;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x)
        keys[off + i] = ((unsigned long long)(stamp[base + i] - stamp_base) << id_bits) | id[base + i];
}

__global__ void unpack_log_kernel(uint32_t n, const unsigned long long* keys, uint32_t stamp_base, uint32_t id_bits,
                                  uint32_t* stamp, uint32_t* id) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const unsigned long long k = keys[i];
        stamp[i] = (uint32_t)(k >> id_bits) + stamp_base;
        id[i] = (uint32_t)(k & ((1ull << id_bits) - 1ull));
    }
}

size_t spike_log_sort_tmp_bytes(uint32_t capacity) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, bytes, (unsigned long long*)nullptr, (unsigned long long*)nullptr,
                                   (int)capacity);
    return bytes + 16;
}

cudaError_t sort_spike_log(uint32_t n, uint32_t* d_stamp, uint32_t* d_id, uint32_t stamp_base, uint32_t stamp_bits,
                           uint32_t id_bits, unsigned long long* d_keys, unsigned long long* d_keys_out, void* tmp,
                           size_t tmp_bytes, cudaStream_t stream, uint32_t n_seg, uint32_t seg_cap, const uint32_t* d_seg_cnt) {
    if (n == 0) return cudaSuccess;
    if (n_seg) pack_log_segments_kernel<<<n_seg, 256, 0, stream>>>(n_seg, seg_cap, d_seg_cnt, d_stamp, d_id, stamp_base, id_bits, d_keys);
    else pack_log_kernel<<<(n + 255) / 256, 256, 0, stream>>>(n, d_stamp, d_id, stamp_base, id_bits, d_keys);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    int end_bit = (int)(stamp_bits + id_bits);
    if (end_bit > 64) end_bit = 64;
    e = cub::DeviceRadixSort::SortKeys(tmp, tmp_bytes, d_keys, d_keys_out, (int)n, 0, end_bit, stream);
    if (e != cudaSuccess) return e;
    unpack_log_kernel<<<(n + 255) / 256, 256, 0, stream>>>(n, d_keys_out, stamp_base, id_bits, d_stamp, d_id);
    return cudaGetLastError();
}

#define CSR_CHECK(x)                      \
    do {                                  \
        cudaError_t e_ = (x);             \
        if (e_ != cudaSuccess) {          \
            err = e_;                     \
            goto done;                    \
        }                                 \
    } while (0)

cudaError_t build_csr_device(uint64_t n_rows, uint64_t n_edges, const uint32_t* h_src, const uint32_t* h_trg,
                             const float* h_w, const uint16_t* h_delay, const uint8_t* h_port, uint32_t lo,
                             uint32_t target_bits, cudaStream_t stream, unsigned long long** d_rowptr_out,
                             uint2** d_entries_out) {
    cudaError_t err = cudaSuccess;
    unsigned long long *d_rowptr = nullptr, *d_keys = nullptr, *d_keys2 = nullptr;
    uint2* d_entries = nullptr;
    uint32_t *d_src = nullptr, *d_trg = nullptr;
    float *d_w = nullptr, *d_w2 = nullptr;
    uint16_t* d_delay = nullptr;
    uint8_t* d_port = nullptr;
    void* d_tmp = nullptr;
    size_t tmp_bytes = 0;
    const int blocks = 148 * 8, threads = 256;

    CSR_CHECK(cudaMalloc(&d_rowptr, sizeof(unsigned long long) * (n_rows + 1)));
    if (n_edges == 0) {
        fill_u64_kernel<<<blocks, threads, 0, stream>>>(d_rowptr, n_rows + 1, 0ull);
        CSR_CHECK(cudaGetLastError());
        CSR_CHECK(cudaMalloc(&d_entries, sizeof(uint2)));
        CSR_CHECK(cudaStreamSynchronize(stream));
        goto done;
    }
    CSR_CHECK(cudaMalloc(&d_src, 4 * n_edges));
    CSR_CHECK(cudaMalloc(&d_trg, 4 * n_edges));
    CSR_CHECK(cudaMalloc(&d_w, 4 * n_edges));
    CSR_CHECK(cudaMalloc(&d_delay, 2 * n_edges));
    CSR_CHECK(cudaMalloc(&d_port, n_edges));
    CSR_CHECK(cudaMalloc(&d_keys, 8 * n_edges));
    CSR_CHECK(cudaMemcpyAsync(d_src, h_src, 4 * n_edges, cudaMemcpyHostToDevice, stream));
    CSR_CHECK(cudaMemcpyAsync(d_trg, h_trg, 4 * n_edges, cudaMemcpyHostToDevice, stream));
    CSR_CHECK(cudaMemcpyAsync(d_w, h_w, 4 * n_edges, cudaMemcpyHostToDevice, stream));
    CSR_CHECK(cudaMemcpyAsync(d_delay, h_delay, 2 * n_edges, cudaMemcpyHostToDevice, stream));
    CSR_CHECK(cudaMemcpyAsync(d_port, h_port, n_edges, cudaMemcpyHostToDevice, stream));
    make_keys_kernel<<<blocks, threads, 0, stream>>>(n_edges, d_src, d_trg, d_delay, d_port, lo, target_bits, d_keys);
    CSR_CHECK(cudaGetLastError());
    CSR_CHECK(cudaStreamSynchronize(stream));
    cudaFree(d_src); d_src = nullptr;
    cudaFree(d_trg); d_trg = nullptr;
    cudaFree(d_delay); d_delay = nullptr;
    cudaFree(d_port); d_port = nullptr;
    CSR_CHECK(cudaMalloc(&d_keys2, 8 * n_edges));
    CSR_CHECK(cudaMalloc(&d_w2, 4 * n_edges));
    {
        int src_bits = 1;
        while (src_bits < 32 && (n_rows >> src_bits) != 0) ++src_bits;
        const int end_bit = 32 + src_bits;
        CSR_CHECK(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_keys, d_keys2, d_w, d_w2, n_edges, 0, end_bit,
                                                  stream));
        CSR_CHECK(cudaMalloc(&d_tmp, tmp_bytes ? tmp_bytes : 16));
        CSR_CHECK(cub::DeviceRadixSort::SortPairs(d_tmp, tmp_bytes, d_keys, d_keys2, d_w, d_w2, n_edges, 0, end_bit,
                                                  stream));
    }
    CSR_CHECK(cudaStreamSynchronize(stream));
    cudaFree(d_tmp); d_tmp = nullptr;
    cudaFree(d_keys); d_keys = nullptr;
    cudaFree(d_w); d_w = nullptr;
    CSR_CHECK(cudaMalloc(&d_entries, sizeof(uint2) * n_edges));
    emit_csr_kernel<<<blocks, threads, 0, stream>>>(n_edges, n_rows, d_keys2, d_w2, d_entries, d_rowptr);
    CSR_CHECK(cudaGetLastError());
    CSR_CHECK(cudaStreamSynchronize(stream));

done:
    cudaFree(d_src); cudaFree(d_trg); cudaFree(d_w); cudaFree(d_delay); cudaFree(d_port);
    cudaFree(d_keys); cudaFree(d_keys2); cudaFree(d_w2); cudaFree(d_tmp);
    if (err != cudaSuccess) {
        cudaFree(d_rowptr);
        cudaFree(d_entries);
        return err;
    }
    *d_rowptr_out = d_rowptr;
    *d_entries_out = d_entries;
    return cudaSuccess;
}

}  // namespace bmtk
