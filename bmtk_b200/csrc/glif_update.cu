// Fused per-step GLIF update (NEST glif_psc semantics, all five mode combinations):
// membrane + after-spike currents + threshold components + alpha-PSC states of four receptor
// ports, ring-slot consume-and-clear, threshold test / refractory reset, spike compaction into
// the window's spike list and the spike log, and the on-line Poisson sources of the step.
//
// Memory plan: structure-of-arrays fp32 state, four neurons per thread, every state array is
// read and written exactly once per step with 128-bit accesses that are contiguous across the
// warp (512 B per warp per array). Algorithmic traffic is 12 state words read + written
// (96 B) plus 4 ring words read + cleared (32 B) = 128 B per neuron-step (+2 B type index).
// Replaces the arithmetic NEST runs inside nest.Simulate
// (bmtk/simulator/pointnet/pointsimulator.py:166).
#include "common.cuh"
#include "glif_math.cuh"
#include "philox.cuh"

namespace bmtk {

constexpr int kUpdateThreads = 128;
constexpr int kNeuronsPerBlock = kUpdateThreads * kNeuronsPerThread;
// Type tables up to this many types are staged in shared memory.
constexpr int kSmemTypes = 128;

template <bool THETA, bool IEXT>
__global__ void __launch_bounds__(kUpdateThreads) glif_update_kernel(const UpdateArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TypeConsts* s_types = reinterpret_cast<TypeConsts*>(smem_raw);
    const bool use_smem = a.n_types <= kSmemTypes;
    const uint32_t neuron_blocks = (a.n_pad + kNeuronsPerBlock - 1) / kNeuronsPerBlock;
    const unsigned long long step = a.ctl->step_base + a.step_in_window;

    if (blockIdx.x >= neuron_blocks) {
        // ---- on-line Poisson virtual cells of this step
        const uint32_t v = (blockIdx.x - neuron_blocks) * kUpdateThreads + threadIdx.x;
        int k = 0;
        uint32_t e = 0;
        if (v < a.n_virtual * a.n_trials) {
            const uint32_t trial = v / a.n_virtual, cell = v - trial * a.n_virtual;
            const uint4 thr = a.poisson_thr[cell];
            const uint32_t x = philox4x32_10(cell, (uint32_t)step, (uint32_t)(step >> 32), a.trial_base + trial,
                                             (uint32_t)a.seed,
                                             (uint32_t)(a.seed >> 32)).x;
            k = (x >= thr.x) + (x >= thr.y) + (x >= thr.z) + (x >= thr.w);
            e = (a.step_in_window << kSrcBits) | (a.ids.n_cells_all + v);
        }
        if (__any_sync(0xffffffffu, k > 0)) {
            uint32_t tot;
            const uint32_t pos = warp_reserve(a.virt, k, &tot);
            for (int j = 0; j < k; ++j) {
                if (pos + j < a.virt_cap) a.virt[1 + pos + j] = e;
                else atomicOr(&a.ctl->error_flags, kErrVirtListFull);
            }
            if ((threadIdx.x & 31) == 31) atomicAdd(&a.ctl->n_input_spikes, (unsigned long long)tot);
        }
        return;
    }

    if (use_smem) {
        const int words = a.n_types * (int)(sizeof(TypeConsts) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.types);
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_types);
        for (int i = threadIdx.x; i < words; i += kUpdateThreads) dst[i] = src[i];
        __syncthreads();
    }
    const TypeConsts* types = use_smem ? s_types : a.types;

    const uint32_t i0 = (blockIdx.x * kUpdateThreads + threadIdx.x) * kNeuronsPerThread;
    uint32_t spk_mask = 0;  // bit j: neuron i0 + j fired in this step
    if (i0 < a.n_pad) {
        const uint32_t np = a.n_pad;
        const uint32_t slot = (uint32_t)(step % a.ring_slots);
        float* ring = a.ring + (size_t)slot * kPorts * np + i0;
        // loads: all independent, issued before any use
        Neuron4<THETA, IEXT> nr;
        nr.load(a.st, np, i0);
        F4 in[kPorts];
#pragma unroll
        for (int p = 0; p < kPorts; ++p) in[p] = ld4(ring + (size_t)p * np);
        spk_mask = nr.step(types, in);
        // cells beyond n_local inside a trial are padding
        const uint32_t li0 = i0 % a.n_pad1;
        if (li0 + kNeuronsPerThread > a.n_local) spk_mask &= (1u << (a.n_local > li0 ? a.n_local - li0 : 0)) - 1u;
        nr.store(a.st, np, i0);
        const F4 zero = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int p = 0; p < kPorts; ++p) st4(ring + (size_t)p * np, zero);
    }

    // spike compaction: one atomic per warp that has spikes
    if (__any_sync(0xffffffffu, spk_mask != 0))
        emit_spikes(spk_mask, (a.step_in_window << kSrcBits) | (a.lo + i0), a.lo + i0, (uint32_t)(step + 1), a.send,
                    a.send_cap, a.ctl, a.log_stamp, a.log_id, a.log_cap);
}

int glif_update_blocks(uint32_t n_pad, uint32_t n_virtual_poisson) {
    return (int)((n_pad + kNeuronsPerBlock - 1) / kNeuronsPerBlock +
                 (n_virtual_poisson + kUpdateThreads - 1) / kUpdateThreads);
}

cudaError_t launch_glif_update(const UpdateArgs& a, bool has_theta, bool has_iext, cudaStream_t s) {
    const int blocks = glif_update_blocks(a.n_pad, a.poisson_thr ? a.n_virtual * a.n_trials : 0);
    if (blocks == 0) return cudaSuccess;
    const size_t smem = a.n_types <= kSmemTypes ? sizeof(TypeConsts) * (size_t)a.n_types : 0;
    if (has_theta) {
        if (has_iext) glif_update_kernel<true, true><<<blocks, kUpdateThreads, smem, s>>>(a);
        else glif_update_kernel<true, false><<<blocks, kUpdateThreads, smem, s>>>(a);
    } else {
        if (has_iext) glif_update_kernel<false, true><<<blocks, kUpdateThreads, smem, s>>>(a);
        else glif_update_kernel<false, false><<<blocks, kUpdateThreads, smem, s>>>(a);
    }
    return cudaGetLastError();
}

}  // namespace bmtk
