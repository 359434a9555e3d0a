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
#include "philox.cuh"

namespace bmtk {

constexpr int kUpdateThreads = 128;
constexpr int kNeuronsPerThread = 4;
constexpr int kNeuronsPerBlock = kUpdateThreads * kNeuronsPerThread;
// Type tables up to this many types are staged in shared memory.
constexpr int kSmemTypes = 128;

struct F4 {
    float v[4];
};
__device__ __forceinline__ F4 ld4(const float* p) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    return F4{{t.x, t.y, t.z, t.w}};
}
__device__ __forceinline__ void st4(float* p, const F4& a) {
    *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
}

// Reserves `n` consecutive positions for this thread behind a shared counter with one atomic per
// warp (inclusive warp scan, lane 31 adds the warp total). Returns the thread's first position;
// *total receives the warp total on every lane. All 32 lanes must call it.
__device__ __forceinline__ uint32_t warp_reserve(uint32_t* counter, int n, uint32_t* total) {
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    int incl = n;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(full, incl, d);
        if (lane >= d) incl += t;
    }
    uint32_t base = 0;
    if (lane == 31) base = atomicAdd(counter, (uint32_t)incl);
    base = __shfl_sync(full, base, 31);
    *total = (uint32_t)__shfl_sync(full, incl, 31);
    return base + (uint32_t)(incl - n);
}

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
        if (v < a.n_virtual) {
            const uint4 thr = a.poisson_thr[v];
            const uint32_t x = philox4x32_10(v, (uint32_t)step, (uint32_t)(step >> 32), 0u, (uint32_t)a.seed,
                                             (uint32_t)(a.seed >> 32)).x;
            k = (x >= thr.x) + (x >= thr.y) + (x >= thr.z) + (x >= thr.w);
            e = (a.step_in_window << kSrcBits) | (a.n_global + v);
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

        // ---- loads (all independent, issued before any use)
        F4 U = ld4(a.st.U + i0), a0 = ld4(a.st.asc0 + i0), a1 = ld4(a.st.asc1 + i0);
        F4 y1[kPorts], y2[kPorts], in[kPorts];
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            y1[p] = ld4(a.st.y1 + (size_t)p * np + i0);
            y2[p] = ld4(a.st.y2 + (size_t)p * np + i0);
            in[p] = ld4(ring + (size_t)p * np);
        }
        const int4 rf4 = *reinterpret_cast<const int4*>(a.st.refr + i0);
        int rf[4] = {rf4.x, rf4.y, rf4.z, rf4.w};
        const ushort4 ty4 = *reinterpret_cast<const ushort4*>(a.st.type + i0);
        const uint16_t ty[4] = {ty4.x, ty4.y, ty4.z, ty4.w};
        F4 ths = {{0, 0, 0, 0}}, thv = {{0, 0, 0, 0}}, iex = {{0, 0, 0, 0}};
        if (THETA) {
            ths = ld4(a.st.th_spike + i0);
            thv = ld4(a.st.th_voltage + i0);
        }
        if (IEXT) iex = ld4(a.st.i_ext + i0);

#pragma unroll
        for (int j = 0; j < kNeuronsPerThread; ++j) {
            const TypeConsts& c = types[ty[j]];
            float u = U.v[j];
            bool spk = false;
            if (rf[j] > 0) {
                // refractory: V is held; the reset happens on the step the countdown ends
                if (--rf[j] == 0) {
                    a0.v[j] = c.asc_amps[0] + a0.v[j] * c.asc_refr[0];
                    a1.v[j] = c.asc_amps[1] + a1.v[j] * c.asc_refr[1];
                    if (THETA && (c.flags & 1)) {
                        u = c.reset_fraction * u + c.reset_add;
                        ths.v[j] = ths.v[j] * c.theta_spike_refr + c.th_spike_add;
                    } else {
                        u = c.v_reset;
                    }
                }
            } else {
                const float asc_sum = c.asc_coeff[0] * a0.v[j] + c.asc_coeff[1] * a1.v[j];
                a0.v[j] *= c.asc_decay[0];
                a1.v[j] *= c.asc_decay[1];
                if (THETA && (c.flags & 1)) ths.v[j] *= c.theta_spike_decay;
                const float v_old = u;
                const float drive = iex.v[j] + asc_sum;
                u = v_old * c.P33 + drive * c.P30;
#pragma unroll
                for (int p = 0; p < kPorts; ++p) u += c.P31[p] * y1[p].v[j] + c.P32[p] * y2[p].v[j];
                float th = c.th_inf;
                if (THETA) {
                    if (c.flags & 2) {
                        const float beta = drive * c.inv_G;
                        const float d = c.phi * (v_old - beta);
                        thv.v[j] = d * c.P33 + c.theta_voltage_decay * (thv.v[j] - d - c.abpara * beta) +
                                   c.abpara * beta;
                    }
                    th += ths.v[j] + thv.v[j];
                }
                if (u > th) {
                    rf[j] = c.n_ref;
                    spk = true;
                }
            }
            U.v[j] = u;
#pragma unroll
            for (int p = 0; p < kPorts; ++p) {
                const float y1o = y1[p].v[j];
                y2[p].v[j] = c.P21[p] * y1o + c.P11[p] * y2[p].v[j];
                y1[p].v[j] = c.P11[p] * y1o + c.psc_init[p] * in[p].v[j];
            }
            if (spk && i0 + j < a.n_local) spk_mask |= 1u << j;
        }

        // ---- stores
        st4(a.st.U + i0, U);
        st4(a.st.asc0 + i0, a0);
        st4(a.st.asc1 + i0, a1);
        const F4 zero = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            st4(a.st.y1 + (size_t)p * np + i0, y1[p]);
            st4(a.st.y2 + (size_t)p * np + i0, y2[p]);
            st4(ring + (size_t)p * np, zero);
        }
        *reinterpret_cast<int4*>(a.st.refr + i0) = make_int4(rf[0], rf[1], rf[2], rf[3]);
        if (THETA) {
            st4(a.st.th_spike + i0, ths);
            st4(a.st.th_voltage + i0, thv);
        }
    }

    // ---- spike compaction: one atomic per warp that has spikes
    const int nspk = __popc(spk_mask);
    if (__any_sync(0xffffffffu, nspk > 0)) {
        const uint32_t ent0 = (a.step_in_window << kSrcBits) | (a.lo + i0);
        uint32_t tot;
        uint32_t pos = warp_reserve(a.send, nspk, &tot);
#pragma unroll
        for (int j = 0; j < kNeuronsPerThread; ++j) {
            if (spk_mask >> j & 1u) {
                if (pos < a.send_cap) a.send[1 + pos] = ent0 + j;
                else atomicOr(&a.ctl->error_flags, kErrSpikeListFull);
                ++pos;
            }
        }
        if ((threadIdx.x & 31) == 31) atomicAdd(&a.ctl->n_spikes, (unsigned long long)tot);
        if (a.log_stamp) {
            // spike log: (stamp = step + 1, global id)
            pos = warp_reserve(&a.ctl->log_count, nspk, &tot);
#pragma unroll
            for (int j = 0; j < kNeuronsPerThread; ++j) {
                if (spk_mask >> j & 1u) {
                    if (pos < a.log_cap) {
                        a.log_stamp[pos] = (uint32_t)(step + 1);
                        a.log_id[pos] = a.lo + i0 + j;
                    } else {
                        atomicOr(&a.ctl->error_flags, kErrLogFull);
                    }
                    ++pos;
                }
            }
        }
    }
}

int glif_update_blocks(uint32_t n_pad, uint32_t n_virtual_poisson) {
    return (int)((n_pad + kNeuronsPerBlock - 1) / kNeuronsPerBlock +
                 (n_virtual_poisson + kUpdateThreads - 1) / kUpdateThreads);
}

cudaError_t launch_glif_update(const UpdateArgs& a, bool has_theta, bool has_iext, cudaStream_t s) {
    const int blocks = glif_update_blocks(a.n_pad, a.poisson_thr ? a.n_virtual : 0);
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
