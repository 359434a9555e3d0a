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

// Sorts the first n entries of the device spike log (d_stamp, d_id) by (stamp, id) in place: packs
// them into keys (stamp - stamp_base) << id_bits | id, radix-sorts (CUB) over the stamp_bits + id_bits
// bits in use and unpacks the sorted keys back into the two arrays. Every stamp must be in
// [stamp_base, stamp_base + 2^stamp_bits) and every id below 2^id_bits. d_keys / d_keys_out hold n keys
// each. With n_seg > 0 the log is kept in n_seg segments of seg_cap entries holding d_seg_cnt[s] entries each
// (n = their sum) and is laid end to end while it is packed. tmp/tmp_bytes is caller-provided scratch of at least spike_log_sort_tmp_bytes(capacity) bytes.
size_t spike_log_sort_tmp_bytes(uint32_t capacity);
cudaError_t sort_spike_log(uint32_t n, uint32_t* d_stamp, uint32_t* d_id, uint32_t stamp_base, uint32_t stamp_bits,
                           uint32_t id_bits, unsigned long long* d_keys, unsigned long long* d_keys_out, void* tmp,
                           size_t tmp_bytes, cudaStream_t stream, uint32_t n_seg = 0, uint32_t seg_cap = 0,
                           const uint32_t* d_seg_cnt = nullptr);

}  // namespace bmtk
