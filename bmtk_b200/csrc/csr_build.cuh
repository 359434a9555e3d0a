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

}  // namespace bmtk
