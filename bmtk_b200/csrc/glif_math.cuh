// Register-resident state of four consecutive neurons and one update step on it.
// Shared by the per-step kernel (state loaded and stored every step) and the persistent kernel
// (state kept in registers across steps).
#pragma once
#include "common.cuh"

namespace bmtk {

constexpr int kNeuronsPerThread = 4;

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

// The constants of a type that the integrating step multiplies and adds, every one twice ({c, c}): the operand form of
// the packed single-precision instructions of sm_100 (fma.rn.f32x2 and friends work on two independent values in a
// 64-bit register pair), read from shared memory with one 64- or 128-bit load. Same members, same order as the head
// of TypeConsts.
struct __align__(16) TypeConsts2 {
    float2 P11[kPorts], P21[kPorts], P31[kPorts], P32[kPorts], psc_init[kPorts];
    float2 asc_decay[2], asc_coeff[2];
    float2 asc_refr[2], asc_amps[2];
    float2 P33, P30, th_inf, i_e;
    float2 v_reset, E_L, inv_G, delta_gain;
};
constexpr int kDupFloats = (int)(sizeof(TypeConsts2) / sizeof(float2));
static_assert(offsetof(TypeConsts2, delta_gain) == 2 * offsetof(TypeConsts, delta_gain) &&
              offsetof(TypeConsts2, asc_amps) == 2 * offsetof(TypeConsts, asc_amps),
              "TypeConsts2 doubles the first kDupFloats floats of TypeConsts");

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

template <bool THETA, bool IEXT>
struct Neuron4 {
    F4 U, a0, a1, y1[kPorts], y2[kPorts], ths, thv, iex;
    int rf[4];
    uint16_t ty[4];

    __device__ __forceinline__ void load(const StateSoA& st, uint32_t np, uint32_t i0) {
        U = ld4(st.U + i0);
        a0 = ld4(st.asc0 + i0);
        a1 = ld4(st.asc1 + i0);
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            y1[p] = ld4(st.y1 + (size_t)p * np + i0);
            y2[p] = ld4(st.y2 + (size_t)p * np + i0);
        }
        const int4 r = *reinterpret_cast<const int4*>(st.refr + i0);
        rf[0] = r.x; rf[1] = r.y; rf[2] = r.z; rf[3] = r.w;
        const ushort4 t = *reinterpret_cast<const ushort4*>(st.type + i0);
        ty[0] = t.x; ty[1] = t.y; ty[2] = t.z; ty[3] = t.w;
        ths = thv = iex = F4{{0.f, 0.f, 0.f, 0.f}};
        if (THETA) {
            ths = ld4(st.th_spike + i0);
            thv = ld4(st.th_voltage + i0);
        }
        if (IEXT) iex = ld4(st.i_ext + i0);
    }

    __device__ __forceinline__ void store(const StateSoA& st, uint32_t np, uint32_t i0) const {
        st4(st.U + i0, U);
        st4(st.asc0 + i0, a0);
        st4(st.asc1 + i0, a1);
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            st4(st.y1 + (size_t)p * np + i0, y1[p]);
            st4(st.y2 + (size_t)p * np + i0, y2[p]);
        }
        *reinterpret_cast<int4*>(st.refr + i0) = make_int4(rf[0], rf[1], rf[2], rf[3]);
        if (THETA) {
            st4(st.th_spike + i0, ths);
            st4(st.th_voltage + i0, thv);
        }
    }

    // Recordable `code` (BMTK_VAR_*) of neuron j after a step.
    __device__ __forceinline__ float probe_value(const TypeConsts& c, int j, uint32_t code) const {
        switch (code) {
            case BMTK_VAR_I_SYN: return __fadd_rn(__fadd_rn(__fadd_rn(y2[0].v[j], y2[1].v[j]), y2[2].v[j]), y2[3].v[j]);
            case BMTK_VAR_ASC_SUM: return __fmaf_rn(c.asc_rec[0], a0.v[j], __fmul_rn(c.asc_rec[1], a1.v[j]));
            case BMTK_VAR_THRESHOLD: return __fadd_rn(__fadd_rn(__fadd_rn(c.th_inf, ths.v[j]), thv.v[j]), c.E_L);
            case BMTK_VAR_TH_SPIKE: return ths.v[j];
            case BMTK_VAR_TH_VOLTAGE: return thv.v[j];
            case BMTK_VAR_I: return __fadd_rn(iex.v[j], c.i_e);
            default: return __fadd_rn(U.v[j], c.E_L);
        }
    }

    // One step of neuron j with ring input in[port][j]; returns whether it fired.
    // Written without branches: both the refractory and the integrating update are evaluated and
    // the result selected, so that the neurons' dependency chains (and their loads of the
    // type constants) interleave instead of running one after the other.
    __device__ __forceinline__ bool step_one(const TypeConsts& c, int j, const F4 (&in)[kPorts]) {
        const float v_old = U.v[j];
        const bool refr = rf[j] > 0;
        const int rf_dec = rf[j] - 1;
        const bool ends = refr && rf_dec == 0;   // glif_psc resets on the step the countdown ends
        const bool sdt = THETA && (c.flags & 1);  // spike-dependent threshold

        // ---- integrating neuron. Every floating-point step below is ONE IEEE-754 single-precision operation in
        // the order written (fused multiply-adds where named so): the compiler may not contract or reorder them,
        // and a CPU restatement with fmaf() reproduces the state bit for bit.
        const float asc_sum = __fmaf_rn(c.asc_coeff[0], a0.v[j], __fmul_rn(c.asc_coeff[1], a1.v[j]));
        const float drive = __fadd_rn(__fadd_rn(iex.v[j], c.i_e), asc_sum);
        float u_int = __fmaf_rn(v_old, c.P33, __fmul_rn(drive, c.P30));
#pragma unroll
        for (int p = 0; p < kPorts; ++p)
            u_int = __fadd_rn(u_int, __fmaf_rn(c.P31[p], y1[p].v[j], __fmul_rn(c.P32[p], y2[p].v[j])));
        // iaf_psc_delta: what arrives in this step is a jump of V (its ports have P31 = P32 = psc_init = 0)
        u_int = __fmaf_rn(c.delta_gain, __fadd_rn(__fadd_rn(in[0].v[j], in[1].v[j]), __fadd_rn(in[2].v[j], in[3].v[j])), u_int);
        const bool fire = finish(c, j, v_old, drive, u_int, refr, ends, rf_dec, sdt);
        a0.v[j] = refr ? (ends ? __fmaf_rn(a0.v[j], c.asc_refr[0], c.asc_amps[0]) : a0.v[j]) : __fmul_rn(a0.v[j], c.asc_decay[0]);
        a1.v[j] = refr ? (ends ? __fmaf_rn(a1.v[j], c.asc_refr[1], c.asc_amps[1]) : a1.v[j]) : __fmul_rn(a1.v[j], c.asc_decay[1]);
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            const float y1o = y1[p].v[j];
            y2[p].v[j] = __fmaf_rn(c.P21[p], y1o, __fmul_rn(c.P11[p], y2[p].v[j]));
            y1[p].v[j] = __fmaf_rn(c.P11[p], y1o, __fmul_rn(c.psc_init[p], in[p].v[j]));
        }
        return fire;
    }

    // What follows the integration of V for neuron j: thresholds, the spike test, and the choice between the
    // integrating and the refractory update of V and the countdown.
    __device__ __forceinline__ bool finish(const TypeConsts& c, int j, float v_old, float drive, float u_int, bool refr, bool ends,
                                           int rf_dec, bool sdt) {
        float th = c.th_inf;
        float ths_int = ths.v[j], thv_int = thv.v[j];
        if (THETA) {
            if (sdt) ths_int = __fmul_rn(ths.v[j], c.theta_spike_decay);
            if (c.flags & 2) {
                const float beta = __fmul_rn(drive, c.inv_G);
                const float d = __fmul_rn(c.phi, __fsub_rn(v_old, beta));
                const float ab = __fmul_rn(c.abpara, beta);
                const float rest = __fsub_rn(__fsub_rn(thv.v[j], d), ab);
                thv_int = __fadd_rn(__fmaf_rn(c.theta_voltage_decay, rest, __fmul_rn(d, c.P33)), ab);
            }
            th = __fadd_rn(th, __fadd_rn(ths_int, thv_int));
        }
        const bool fire = !refr && ((c.flags & 8) ? (u_int >= th) : (u_int > th));
        if ((c.flags & 4) && fire) u_int = c.v_reset;   // iaf_psc_alpha: reset in the spike step

        // ---- refractory neuron: V is held; after-spike currents and V change when the countdown ends
        const float u_end = sdt ? __fmaf_rn(c.reset_fraction, v_old, c.reset_add) : c.v_reset;

        U.v[j] = refr ? (ends ? u_end : v_old) : u_int;
        if (THETA) {
            ths.v[j] = refr ? ((ends && sdt) ? __fmaf_rn(ths.v[j], c.theta_spike_refr, c.th_spike_add) : ths.v[j]) : ths_int;
            thv.v[j] = refr ? thv.v[j] : thv_int;
        }
        rf[j] = refr ? rf_dec : (fire ? c.n_ref : rf[j]);
        return fire;
    }

    // One step for the four neurons with ring input in[port]. Returns the spike mask (bit j).
    __device__ __forceinline__ uint32_t step(const TypeConsts* types, const F4 (&in)[kPorts]) {
        uint32_t mask = 0;
#pragma unroll
        for (int j = 0; j < kNeuronsPerThread; ++j) mask |= step_one(types[ty[j]], j, in) ? (1u << j) : 0u;
        return mask;
    }

    // The same step for neurons j and j + 1 of ONE type with the packed single-precision instructions: every
    // operation of step_one is done for both neurons by one instruction (element-wise IEEE-754, so the bits are
    // those of step_one), with the constants taken doubled from `d`.
    __device__ __forceinline__ uint32_t step_pair(const TypeConsts& c, const TypeConsts2& d, int j, const F4 (&in)[kPorts]) {
        const int k = j + 1;
        const float2 v_old = f2(U.v[j], U.v[k]), a0p = f2(a0.v[j], a0.v[k]), a1p = f2(a1.v[j], a1.v[k]);
        const float2 asc_sum = __ffma2_rn(d.asc_coeff[0], a0p, __fmul2_rn(d.asc_coeff[1], a1p));
        const float2 drive = __fadd2_rn(__fadd2_rn(f2(iex.v[j], iex.v[k]), d.i_e), asc_sum);
        float2 u = __ffma2_rn(v_old, d.P33, __fmul2_rn(drive, d.P30));
#pragma unroll
        for (int p = 0; p < kPorts; ++p)
            u = __fadd2_rn(u, __ffma2_rn(d.P31[p], f2(y1[p].v[j], y1[p].v[k]), __fmul2_rn(d.P32[p], f2(y2[p].v[j], y2[p].v[k]))));
        u = __ffma2_rn(d.delta_gain, __fadd2_rn(__fadd2_rn(f2(in[0].v[j], in[0].v[k]), f2(in[1].v[j], in[1].v[k])),
                                                __fadd2_rn(f2(in[2].v[j], in[2].v[k]), f2(in[3].v[j], in[3].v[k]))), u);
        const bool sdt = THETA && (c.flags & 1);
        const bool refr_j = rf[j] > 0, refr_k = rf[k] > 0;
        const int dec_j = rf[j] - 1, dec_k = rf[k] - 1;
        const bool ends_j = refr_j && dec_j == 0, ends_k = refr_k && dec_k == 0;
        const bool fire_j = finish(c, j, v_old.x, drive.x, u.x, refr_j, ends_j, dec_j, sdt);
        const bool fire_k = finish(c, k, v_old.y, drive.y, u.y, refr_k, ends_k, dec_k, sdt);
        {
            const float2 a_refr = __ffma2_rn(a0p, d.asc_refr[0], d.asc_amps[0]), a_dec = __fmul2_rn(a0p, d.asc_decay[0]);
            a0.v[j] = refr_j ? (ends_j ? a_refr.x : a0p.x) : a_dec.x;
            a0.v[k] = refr_k ? (ends_k ? a_refr.y : a0p.y) : a_dec.y;
        }
        {
            const float2 a_refr = __ffma2_rn(a1p, d.asc_refr[1], d.asc_amps[1]), a_dec = __fmul2_rn(a1p, d.asc_decay[1]);
            a1.v[j] = refr_j ? (ends_j ? a_refr.x : a1p.x) : a_dec.x;
            a1.v[k] = refr_k ? (ends_k ? a_refr.y : a1p.y) : a_dec.y;
        }
#pragma unroll
        for (int p = 0; p < kPorts; ++p) {
            const float2 y1o = f2(y1[p].v[j], y1[p].v[k]);
            const float2 n2 = __ffma2_rn(d.P21[p], y1o, __fmul2_rn(d.P11[p], f2(y2[p].v[j], y2[p].v[k])));
            const float2 n1 = __ffma2_rn(d.P11[p], y1o, __fmul2_rn(d.psc_init[p], f2(in[p].v[j], in[p].v[k])));
            y2[p].v[j] = n2.x; y2[p].v[k] = n2.y;
            y1[p].v[j] = n1.x; y1[p].v[k] = n1.y;
        }
        return (fire_j ? (1u << j) : 0u) | (fire_k ? (1u << k) : 0u);
    }

    // One step for the four neurons, pairwise packed where the two neurons of a pair are of one type (neurons are
    // sorted by type: all pairs but those that straddle a boundary between types).
    __device__ __forceinline__ uint32_t step_packed(const TypeConsts* types, const TypeConsts2* types2, const F4 (&in)[kPorts]) {
        uint32_t mask = 0;
#pragma unroll
        for (int j = 0; j < kNeuronsPerThread; j += 2) {
            if (ty[j] == ty[j + 1]) {
                mask |= step_pair(types[ty[j]], types2[ty[j]], j, in);
            } else {
                mask |= step_one(types[ty[j]], j, in) ? (1u << j) : 0u;
                mask |= step_one(types[ty[j + 1]], j + 1, in) ? (2u << j) : 0u;
            }
        }
        return mask;
    }
};

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

// Appends the fired neurons of this thread (mask over i0..i0+3) to the window spike list and, when
// recording, to the spike log. Must be called by all lanes of a warp when any lane has a spike.
__device__ __forceinline__ void emit_spikes(uint32_t spk_mask, uint32_t ent0, uint32_t gid0, uint32_t stamp,
                                            uint32_t* list, uint32_t cap, Ctl* ctl, uint32_t* log_stamp,
                                            uint32_t* log_id, uint32_t log_cap) {
    const int nspk = __popc(spk_mask);
    uint32_t tot;
    uint32_t pos = warp_reserve(list, nspk, &tot);
#pragma unroll
    for (int j = 0; j < kNeuronsPerThread; ++j) {
        if (spk_mask >> j & 1u) {
            if (pos < cap) list[1 + pos] = ent0 + j;
            else atomicOr(&ctl->error_flags, kErrSpikeListFull);
            ++pos;
        }
    }
    if ((threadIdx.x & 31) == 31) atomicAdd(&ctl->n_spikes, (unsigned long long)tot);
    if (log_stamp) {
        pos = warp_reserve(&ctl->log_count, nspk, &tot);
#pragma unroll
        for (int j = 0; j < kNeuronsPerThread; ++j) {
            if (spk_mask >> j & 1u) {
                if (pos < log_cap) {
                    log_stamp[pos] = stamp;
                    log_id[pos] = gid0 + j;
                } else {
                    atomicOr(&ctl->error_flags, kErrLogFull);
                }
                ++pos;
            }
        }
    }
}

}  // namespace bmtk
