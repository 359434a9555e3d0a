#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace bmtk {

// Scratch of the deterministic propagation path (allocated once, sized by capacities).
struct DetWorkspace {
    unsigned long long *item_keys = nullptr, *item_keys2 = nullptr;  // (emit step << 32 | source row)
    uint32_t *row_len = nullptr, *row_off = nullptr;
    uint32_t *ev_key = nullptr, *ev_key2 = nullptr;                  // ring cell index per event
    float *ev_val = nullptr, *ev_val2 = nullptr;
    void* cub_tmp = nullptr;
    size_t cub_tmp_bytes = 0;
    uint32_t item_cap = 0, event_cap = 0;
    int cell_bits = 32;
    uint32_t* h_pinned = nullptr;  // two words read back per window
};

cudaError_t det_alloc(DetWorkspace& w, uint32_t event_cap, uint32_t item_cap, uint64_t ring_cells);
void det_free(DetWorkspace& w);

// One window of deterministic delivery: returns 0, -1 (CUDA error) or -2 (capacity exceeded).
int propagate_det_window(const PropArgs& a, DetWorkspace& w, cudaStream_t s, uint64_t* launches);

}  // namespace bmtk
