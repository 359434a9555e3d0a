#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bmtk {

// Sorts the host edge list into the delay-bucketed CSR on the current device.
// On success *d_rowptr_out ([n_rows+1]) and *d_entries_out ([max(n_edges,1)]) are cudaMalloc'd
// buffers owned by the caller.
cudaError_t build_csr_device(uint64_t n_rows, uint64_t n_edges, const uint32_t* h_src, const uint32_t* h_trg,
                             const float* h_w, const uint16_t* h_delay, const uint8_t* h_port, uint32_t lo,
                             uint32_t target_bits, cudaStream_t stream, unsigned long long** d_rowptr_out,
                             uint2** d_entries_out);

// Sorts the first n entries of the device spike log by (stamp, id): packs them into 64-bit keys,
// radix-sorts (CUB) and leaves the sorted keys (stamp << 32 | id) in d_keys_out. tmp/tmp_bytes is
// caller-provided scratch of at least spike_log_sort_tmp_bytes(capacity) bytes.
size_t spike_log_sort_tmp_bytes(uint32_t capacity);
cudaError_t sort_spike_log(uint32_t n, const uint32_t* d_stamp, const uint32_t* d_id, unsigned long long* d_keys,
                           unsigned long long* d_keys_out, void* tmp, size_t tmp_bytes, cudaStream_t stream);

}  // namespace bmtk
