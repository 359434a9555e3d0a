#pragma once
#include "persistent.cuh"

namespace bmtk {

constexpr uint32_t kPipeMaxBlocks = 512;    // largest grid (one block per SM)
constexpr uint32_t kPipeSegCap = 1024;      // chunk descriptors one block can add to one phase's list

// Pipelined persistent kernel (update and delivery warps side by side on every SM). Takes the
// same arguments as the two-phase persistent kernel plus PersistArgs::half, the phase length.
size_t pipelined_smem(int n_types, uint32_t chunk_warps, uint32_t ring_stage_warps = 0);
uint32_t pipelined_max_update_warps();   // a block can hold this many update warps of 128 neurons
uint32_t pipelined_warps();              // warps of a block: update + delivery
uint32_t pipelined_warps_small();        // ... of the small block (more registers per thread)
int pipelined_max_blocks(int device, bool has_theta, bool has_iext, size_t smem);
cudaError_t launch_pipelined(const PersistArgs& a, bool has_theta, bool has_iext, int blocks, cudaStream_t s);

}  // namespace bmtk
