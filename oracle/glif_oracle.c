/*
 * CPU oracle for the point-neuron hot path (TEST INFRASTRUCTURE, not product).
 *
 * A plain-C, fp64 restatement of what BMTK's PointNet asks NEST to do between
 * nest.Simulate() entering and returning (bmtk/simulator/pointnet/pointsimulator.py:166):
 *   - the per-step update of NEST model `glif_psc` (chosen by
 *     examples/point_450glifs/network/v1_node_types.csv, model_template nest:glif_psc;
 *     parameters as produced by bmtk/simulator/pointnet/glif_utils.py:259-418),
 *   - static_synapse spike delivery into per-receptor ring buffers
 *     (connections made at bmtk/simulator/pointnet/pointnetwork.py:229-248),
 *   - spike_generator replay of virtual cells (pointnetwork.py:52-61,187-227),
 *   - step_current_generator clamps attached with delay = dt
 *     (bmtk/simulator/pointnet/modules/iclamp.py:42-54).
 *
 * NEST itself (pinned nest-simulator=3.3, docker/environment.yml:15) is a third-party
 * dependency that is not part of the reference tree, so the arithmetic below restates the
 * published algorithm of its glif_psc model (exact integration of the linear sub-threshold
 * system, Rotter & Diesmann 1999; GLIF rules of Teeter et al. 2018) in the model's own
 * update order:
 *   refractory neurons hold V and are reset when the countdown ends; otherwise
 *   V <- V*P33 + (I + sum_j c_j*ASC_j)*P30 + sum_p (P31_p*y1_p + P32_p*y2_p),
 *   ASC_j <- ASC_j*exp(-k_j h), strict `>` threshold test, then for every neuron
 *   y2_p <- h*e^{-h/tau_p}*y1_p + e^{-h/tau_p}*y2_p, y1_p <- e^{-h/tau_p}*y1_p + (e/tau_p)*ring_p[n],
 *   and finally the clamp current for the next step is latched.
 * The only numeric anchor to real NEST output that the reference holds is the known-answer
 * test bmtk/tests/simulator/pointnet/test_glif_utils.py:16-44 (spike count exact, times
 * atol 1.0 ms); tests/test_oracle_golden.py pins this file against it. Beyond that test,
 * PARITY WITH NEST IS UNPINNED.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu-baseline legs may load this file's
 * shared object. The product (bmtk_b200/) never does.
 *
 * Time grid: step n advances t_n = n*h to t_{n+1}. A spike emitted while executing step n
 * is stamped (n+1)*h; through a synapse of d steps it is consumed by the target at the end
 * of step n+d (ring slot (n+d) mod S), i.e. it first moves V in step n+d+2 via y2.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MAX_PORTS 4

/* NEST glif_psc parameter names (NEST-format dynamics_params JSON, e.g.
 * examples/point_components/cell_models/593618144_glif_lif_asc_psc.json). */
typedef struct {
    double V_m, V_th, g, E_L, C_m, t_ref, V_reset;
    double asc_init[2], asc_decay[2], asc_amps[2], asc_r[2];
    double tau_syn[ORC_MAX_PORTS];
    double th_spike_add, th_spike_decay, voltage_reset_fraction, voltage_reset_add;
    double th_voltage_index, th_voltage_decay;
    int32_t n_ports;
    int32_t spike_dependent_threshold, after_spike_currents, adapting_threshold;
    double I_e;
    int32_t model;      /* 0 glif_psc, 1 iaf_psc_alpha, 2 iaf_psc_delta */
    int32_t reserved;
} orc_glif_params;

/* Per-type constants for one resolution h. */
typedef struct {
    double P33, P30;
    double P11[ORC_MAX_PORTS], P21[ORC_MAX_PORTS], P31[ORC_MAX_PORTS], P32[ORC_MAX_PORTS];
    double psc_init[ORC_MAX_PORTS];
    double asc_decay_rate[2], asc_stable_coeff[2], asc_refr_rate[2], asc_amps[2];
    double th_inf, v_reset;            /* relative to E_L */
    double theta_spike_decay, theta_spike_refr_decay, th_spike_add;
    double reset_fraction, reset_add;
    double phi, abpara, theta_voltage_decay, G;
    double E_L;
    int32_t n_ref;                     /* update steps from spike to reset, inclusive */
    int32_t n_ports, has_theta_spike, has_asc, has_theta_voltage;
    double I_e;
    int32_t iaf;                       /* iaf_psc_alpha / iaf_psc_delta conventions: reset in the spike step, >= test */
    int32_t delta;                     /* iaf_psc_delta: arriving weights are jumps of V, no PSC states */
} orc_glif_consts;

/* x + expm1(-x), accurate for small |x| (the numerator of the alpha-kernel/membrane cross term). */
static double x_plus_expm1_neg(double x)
{
    if (fabs(x) < 1e-3) {
        /* x^2/2 - x^3/6 + x^4/24 - x^5/120 + x^6/720 */
        return x * x * (0.5 + x * (-1.0 / 6.0 + x * (1.0 / 24.0 + x * (-1.0 / 120.0 + x / 720.0))));
    }
    return x + expm1(-x);
}

/* Number of update steps a neuron stays refractory: NEST sets a double countdown to t_ref
 * at the spike and subtracts h once per following step until it is <= 0. The floating-point
 * countdown is reproduced literally so that e.g. t_ref = 2.0, h = 0.1 gives the same count. */
static int32_t refractory_steps(double t_ref, double h)
{
    double r = t_ref;
    int32_t n = 0;
    do {
        r -= h;
        ++n;
    } while (r > 0.0 && n < (1 << 30));
    return n;
}

void orc_glif_consts_init(const orc_glif_params* p, double h, orc_glif_consts* c)
{
    memset(c, 0, sizeof(*c));
    const double tau = p->C_m / p->g;
    c->n_ports = p->n_ports;
    c->has_theta_spike = p->spike_dependent_threshold;
    c->has_asc = p->after_spike_currents;
    c->has_theta_voltage = p->adapting_threshold;
    c->E_L = p->E_L;
    c->G = p->g;
    c->P33 = exp(-h / tau);
    c->P30 = -expm1(-h / tau) / p->g; /* (1 - P33) * tau / C_m */
    for (int k = 0; k < p->n_ports; ++k) {
        const double ts = p->tau_syn[k];
        const double a = 1.0 / ts, b = 1.0 / tau, cc = b - a;
        const double ea = exp(-a * h);
        c->P11[k] = ea;
        c->P21[k] = h * ea;
        c->psc_init[k] = M_E / ts;
        /* dU/dt = -U/tau + y2/C, y2' = y1 - y2/ts, y1' = -y1/ts over one step:
         *   P32 = (e^{-ah} - e^{-bh}) / (c C)            -> h e^{-bh}/C        as c -> 0
         *   P31 = [h e^{-ah}/c - (e^{-ah}-e^{-bh})/c^2]/C -> h^2 e^{-bh}/(2C)  as c -> 0 */
        const double x = cc * h;
        if (x == 0.0) {
            c->P32[k] = h * exp(-b * h) / p->C_m;
            c->P31[k] = 0.5 * h * h * exp(-b * h) / p->C_m;
        } else {
            c->P32[k] = ea * (-expm1(-x)) / (cc * p->C_m);
            c->P31[k] = ea * x_plus_expm1_neg(x) / (cc * cc * p->C_m);
        }
    }
    for (int j = 0; j < 2; ++j) {
        const double k = p->asc_decay[j];
        c->asc_decay_rate[j] = exp(-k * h);
        c->asc_stable_coeff[j] = -expm1(-k * h) / (k * h); /* mean of the decaying ASC over the step */
        c->asc_refr_rate[j] = p->asc_r[j] * exp(-k * p->t_ref);
        c->asc_amps[j] = p->asc_amps[j];
    }
    c->th_inf = p->V_th - p->E_L;
    c->v_reset = p->V_reset - p->E_L;
    c->n_ref = refractory_steps(p->t_ref, h);
    c->I_e = p->I_e;
    c->iaf = p->model == 1 || p->model == 2;
    c->delta = p->model == 2;
    if (c->delta) {
        /* NEST iaf_psc_delta: y3 <- P30 (y0 + I_e) + P33 y3 + spikes.get_value(lag) while not refractory; input
         * that arrives during the refractory period is read and dropped (refractory_input = false);
         * one receptor, excitatory and inhibitory weights share it. Used by
         * examples/point_120cells/network/cortex_node_types.csv:2-3. */
        c->n_ports = 0;
    }
    if (c->iaf) {
        /* NEST iaf_psc_alpha: RefractoryCounts = Time(ms(t_ref)).get_steps(); V is set to V_reset in
         * the spike step and not integrated for that many following steps; spike when V >= V_th. */
        c->n_ref = (int32_t)llround(p->t_ref / h);
        if (c->n_ref < 1) c->n_ref = 1;
    }
    c->theta_spike_decay = exp(-p->th_spike_decay * h);
    c->theta_spike_refr_decay = exp(-p->th_spike_decay * p->t_ref);
    c->th_spike_add = p->th_spike_add;
    c->reset_fraction = p->voltage_reset_fraction;
    c->reset_add = p->voltage_reset_add;
    if (p->adapting_threshold) {
        c->theta_voltage_decay = exp(-p->th_voltage_decay * h);
        c->phi = p->th_voltage_index / (p->th_voltage_decay - p->g / p->C_m);
        c->abpara = p->th_voltage_index / p->th_voltage_decay;
    }
}

/* Everything one run needs; arrays are caller-owned. Neuron ids are 0..n_neurons-1, virtual
 * (spike-replay) sources are n_neurons..n_neurons+n_virtual-1 and only appear as CSR rows. */
typedef struct {
    /* nodes */
    int64_t n_neurons, n_virtual;
    const int32_t* type_index;          /* [n_neurons] */
    int32_t n_types;
    const orc_glif_params* types;       /* [n_types] */
    /* edges, CSR by source (rows: neurons then virtual sources) */
    const int64_t* rowptr;              /* [n_neurons + n_virtual + 1] */
    const int32_t* target;              /* [E] */
    const int32_t* port;                /* [E] 0-based */
    const int32_t* delay;               /* [E] steps, >= 1 */
    const double* weight;               /* [E] pA */
    int32_t max_delay;
    /* replayed virtual spikes, grouped by emitting step: a spike stamped T steps is emitted in
     * step T-1 (spike_generator semantics) */
    const int64_t* in_step_ptr;         /* [n_steps_total + 1] or NULL */
    const int32_t* in_src;              /* virtual index 0..n_virtual-1 */
    /* clamp events: at the START of step `ce_step` the target's external current changes by delta */
    int64_t n_clamp;
    const int64_t* ce_step;             /* sorted ascending */
    const int32_t* ce_target;
    const double* ce_delta;
    /* run */
    double dt;
    int64_t step0, n_steps;             /* run steps step0 .. step0+n_steps-1 */
    int32_t n_threads;
    /* state (in/out), all [n_neurons] except y1,y2 [ORC_MAX_PORTS*n_neurons] (port-major) and
     * ring [S*ORC_MAX_PORTS*n_neurons] with S = max_delay+1 */
    double *U, *asc, *y1, *y2, *th_spike, *th_voltage, *i_ext, *ring;
    int32_t* refr;
    /* outputs */
    int64_t spike_cap;
    int64_t* n_spikes;                  /* in/out running count */
    int64_t* spike_step;                /* stamp in steps (n+1) */
    int32_t* spike_id;
    int32_t n_probe;
    const int32_t* probe_ids;
    int32_t probe_interval;             /* steps */
    double* trace;                      /* [samples][n_probe_vars][n_probe], after the step ending at k*interval */
    int64_t* n_samples;                 /* in/out running count */
    int64_t* n_events;                  /* in/out: synaptic events delivered */
    /* recorded variables (NEST multimeter `record_from`, bmtk/simulator/pointnet/modules/multimeter_reporter.py:103-115):
     * count (0 = V_m only) and codes, 4 bits each: 0 V_m, 1 I_syn = sum of the ports' PSCs y2, 2 ASCurrents_sum = the
     * step mean sum_j c_j ASC_j the latest integrating step used, stated from the current values as
     * sum_j (c_j / decay_j) ASC_j (exact except in the sample at which the refractory period ends), 3 threshold =
     * V_th + spike + voltage component (absolute mV), 4 threshold_spike, 5 threshold_voltage, 6 I = I_e + clamp current */
    int32_t n_probe_vars;
    uint32_t probe_vars;
} orc_run_args;

int64_t orc_state_ring_slots(int32_t max_delay) { return (int64_t)max_delay + 1; }

/* Initial state for every neuron: V = V_m, ASC = asc_init, PSC states 0 (glif_psc defaults). */
void orc_init_state(const orc_run_args* a)
{
    const int64_t N = a->n_neurons;
    for (int64_t i = 0; i < N; ++i) {
        const orc_glif_params* p = &a->types[a->type_index[i]];
        a->U[i] = p->V_m - p->E_L;
        a->asc[i] = p->asc_init[0];
        a->asc[N + i] = p->asc_init[1];
        a->th_spike[i] = 0.0;
        a->th_voltage[i] = 0.0;
        a->i_ext[i] = 0.0;
        a->refr[i] = 0;
    }
    memset(a->y1, 0, sizeof(double) * ORC_MAX_PORTS * N);
    memset(a->y2, 0, sizeof(double) * ORC_MAX_PORTS * N);
    memset(a->ring, 0, sizeof(double) * orc_state_ring_slots(a->max_delay) * ORC_MAX_PORTS * N);
}

static void deliver_row(const orc_run_args* a, int64_t src, int64_t n, int64_t S, int parallel)
{
    const int64_t N = a->n_neurons;
    const int64_t b = a->rowptr[src], e = a->rowptr[src + 1];
    for (int64_t k = b; k < e; ++k) {
        const int64_t slot = (n + a->delay[k]) % S;
        double* cell = &a->ring[(slot * ORC_MAX_PORTS + a->port[k]) * N + a->target[k]];
        if (parallel) {
#pragma omp atomic
            *cell += a->weight[k];
        } else {
            *cell += a->weight[k];
        }
    }
}

int orc_run(orc_run_args* a)
{
    const int64_t N = a->n_neurons;
    const int64_t S = orc_state_ring_slots(a->max_delay);
    const double h = a->dt;
    orc_glif_consts* C = (orc_glif_consts*)malloc(sizeof(orc_glif_consts) * (size_t)a->n_types);
    uint8_t* fired = (uint8_t*)malloc((size_t)(N > 0 ? N : 1));
    if (!C || !fired) { free(C); free(fired); return -1; }
    for (int t = 0; t < a->n_types; ++t) orc_glif_consts_init(&a->types[t], h, &C[t]);
    int nthreads = a->n_threads > 0 ? a->n_threads : 1;
#ifdef _OPENMP
    omp_set_num_threads(nthreads);
#else
    nthreads = 1;
#endif
    const int parallel = nthreads > 1;
    int64_t ce = 0;
    while (ce < a->n_clamp && a->ce_step[ce] < a->step0) ++ce;
    int status = 0;

    for (int64_t n = a->step0; n < a->step0 + a->n_steps; ++n) {
        /* clamp changes that become effective for this step */
        while (ce < a->n_clamp && a->ce_step[ce] == n) {
            a->i_ext[a->ce_target[ce]] += a->ce_delta[ce];
            ++ce;
        }
        const int64_t slot = n % S;
#pragma omp parallel for schedule(static) if (parallel)
        for (int64_t i = 0; i < N; ++i) {
            const orc_glif_consts* c = &C[a->type_index[i]];
            double U = a->U[i];
            uint8_t spk = 0;
            if (a->refr[i] > 0) {
                if (--a->refr[i] == 0) {
                    if (c->has_asc) {
                        a->asc[i] = c->asc_amps[0] + a->asc[i] * c->asc_refr_rate[0];
                        a->asc[N + i] = c->asc_amps[1] + a->asc[N + i] * c->asc_refr_rate[1];
                    }
                    if (!c->has_theta_spike) {
                        U = c->v_reset;
                    } else {
                        U = c->reset_fraction * U + c->reset_add;
                        a->th_spike[i] = a->th_spike[i] * c->theta_spike_refr_decay + c->th_spike_add;
                    }
                }
            } else {
                double asc_sum = 0.0;
                if (c->has_asc) {
                    asc_sum = c->asc_stable_coeff[0] * a->asc[i] + c->asc_stable_coeff[1] * a->asc[N + i];
                    a->asc[i] *= c->asc_decay_rate[0];
                    a->asc[N + i] *= c->asc_decay_rate[1];
                }
                if (c->has_theta_spike) a->th_spike[i] *= c->theta_spike_decay;
                const double v_old = U;
                const double I = a->i_ext[i] + c->I_e;
                U = v_old * c->P33 + (I + asc_sum) * c->P30;
                for (int p = 0; p < c->n_ports; ++p)
                    U += c->P31[p] * a->y1[p * N + i] + c->P32[p] * a->y2[p * N + i];
                if (c->delta) {
                    double jump = 0.0;
                    for (int p = 0; p < ORC_MAX_PORTS; ++p) jump += a->ring[(slot * ORC_MAX_PORTS + p) * N + i];
                    U += jump;
                }
                if (c->has_theta_voltage) {
                    const double beta = (I + asc_sum) / c->G;
                    const double d = c->phi * (v_old - beta);
                    a->th_voltage[i] = d * c->P33
                        + c->theta_voltage_decay * (a->th_voltage[i] - d - c->abpara * beta)
                        + c->abpara * beta;
                }
                const double th = a->th_spike[i] + a->th_voltage[i] + c->th_inf;
                if (c->iaf ? (U >= th) : (U > th)) {
                    a->refr[i] = c->n_ref;
                    spk = 1;
                    if (c->iaf) U = c->v_reset;
                }
            }
            a->U[i] = U;
            fired[i] = spk;
            for (int p = 0; p < c->n_ports; ++p) {
                double* cell = &a->ring[(slot * ORC_MAX_PORTS + p) * N + i];
                const double y1 = a->y1[p * N + i];
                a->y2[p * N + i] = c->P21[p] * y1 + c->P11[p] * a->y2[p * N + i];
                a->y1[p * N + i] = c->P11[p] * y1 + c->psc_init[p] * (*cell);
                *cell = 0.0;
            }
            if (c->delta)
                for (int p = 0; p < ORC_MAX_PORTS; ++p) a->ring[(slot * ORC_MAX_PORTS + p) * N + i] = 0.0;
        }
        /* record + deliver, in ascending neuron id then virtual sources */
        for (int64_t i = 0; i < N; ++i) {
            if (!fired[i]) continue;
            if (a->spike_step) {
                if (*a->n_spikes < a->spike_cap) {
                    a->spike_step[*a->n_spikes] = n + 1;
                    a->spike_id[*a->n_spikes] = (int32_t)i;
                } else {
                    status = 1; /* spike log full: later spikes are counted but not stored */
                }
            }
            ++*a->n_spikes;
        }
        if (parallel) {
            int64_t ev = 0;
#pragma omp parallel for schedule(dynamic, 16) reduction(+ : ev)
            for (int64_t i = 0; i < N; ++i) {
                if (!fired[i]) continue;
                deliver_row(a, i, n, S, 1);
                ev += a->rowptr[i + 1] - a->rowptr[i];
            }
            *a->n_events += ev;
        } else {
            for (int64_t i = 0; i < N; ++i) {
                if (!fired[i]) continue;
                deliver_row(a, i, n, S, 0);
                *a->n_events += a->rowptr[i + 1] - a->rowptr[i];
            }
        }
        if (a->in_step_ptr) {
            for (int64_t k = a->in_step_ptr[n]; k < a->in_step_ptr[n + 1]; ++k) {
                const int64_t src = N + a->in_src[k];
                deliver_row(a, src, n, S, 0);
                *a->n_events += a->rowptr[src + 1] - a->rowptr[src];
            }
        }
        if (a->n_probe > 0 && a->probe_interval > 0 && (n + 1) % a->probe_interval == 0) {
            const int nv = a->n_probe_vars > 0 ? a->n_probe_vars : 1;
            double* row = a->trace + (*a->n_samples) * a->n_probe * nv;
            for (int v = 0; v < nv; ++v) {
                const uint32_t code = a->n_probe_vars > 0 ? (a->probe_vars >> (4 * v)) & 15u : 0u;
                for (int q = 0; q < a->n_probe; ++q) {
                    const int32_t i = a->probe_ids[q];
                    const orc_glif_consts* c = &C[a->type_index[i]];
                    double x;
                    switch (code) {
                        case 1: x = 0.0; for (int p = 0; p < c->n_ports; ++p) x += a->y2[p * N + i]; break;
                        case 2:
                            x = c->has_asc ? c->asc_stable_coeff[0] / c->asc_decay_rate[0] * a->asc[i]
                                             + c->asc_stable_coeff[1] / c->asc_decay_rate[1] * a->asc[N + i] : 0.0;
                            break;
                        case 3: x = c->th_inf + a->th_spike[i] + a->th_voltage[i] + c->E_L; break;
                        case 4: x = a->th_spike[i]; break;
                        case 5: x = a->th_voltage[i]; break;
                        case 6: x = a->i_ext[i] + c->I_e; break;
                        default: x = a->U[i] + c->E_L;
                    }
                    row[v * a->n_probe + q] = x;
                }
            }
            ++*a->n_samples;
        }
    }
    free(C);
    free(fired);
    return status;
}

/* ---- Philox4x32-10 (Salmon et al., SC'11), the counter-based generator of the on-line
 * Poisson sources. counter = (source, step_lo, step_hi, stream), key = (seed_lo, seed_hi). */
void orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* Poisson count for one (source, step) by CDF inversion on the raw 32-bit draw x0:
 * count = #{k in 0..3 : x0 >= T_k}, T_k = floor(2^32 * P[X <= k]) (fp64, clamped to 2^32-1).
 * Integer thresholds keep host and device bit-identical; the count is truncated at 4, which
 * for lambda = rate*dt <= 0.25 happens with probability < 1e-5 per draw. */
void orc_poisson_thresholds(double lambda, uint32_t thr[4])
{
    double p = exp(-lambda), cdf = 0.0;
    for (int k = 0; k < 4; ++k) {
        cdf += p;
        const double t = floor(cdf * 4294967296.0);
        thr[k] = t >= 4294967295.0 ? 0xFFFFFFFFu : (uint32_t)t;
        p *= lambda / (double)(k + 1);
    }
}

int32_t orc_poisson_count_stream(uint32_t source, uint64_t step, uint32_t stream, uint64_t seed, const uint32_t thr[4])
{
    /* counter = (source, step lo, step hi, stream): stream is the trial of a trial-batched run */
    const uint32_t ctr[4] = { source, (uint32_t)step, (uint32_t)(step >> 32), stream };
    const uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
    uint32_t out[4];
    orc_philox4x32_10(ctr, key, out);
    int32_t k = 0;
    for (int j = 0; j < 4; ++j) k += out[0] >= thr[j];
    return k;
}

int32_t orc_poisson_count(uint32_t source, uint64_t step, uint64_t seed, const uint32_t thr[4])
{
    const uint32_t ctr[4] = { source, (uint32_t)step, (uint32_t)(step >> 32), 0u };
    const uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
    uint32_t out[4];
    orc_philox4x32_10(ctr, key, out);
    int32_t k = 0;
    for (int j = 0; j < 4; ++j) k += out[0] >= thr[j];
    return k;
}

/* All Poisson spikes of steps [step0, step0+n_steps) for n_virtual sources with per-source
 * thresholds thr[4*v..4*v+3], ordered by (step, source); a count of k gives k entries.
 * Returns the number of spikes (entries beyond cap are counted, not stored). */
int64_t orc_poisson_fill_stream(int64_t n_virtual, const uint32_t* thr, uint64_t seed, uint32_t stream, int64_t step0,
                                int64_t n_steps, int64_t cap, int64_t* emit_step, int32_t* source)
{
    int64_t n = 0;
    for (int64_t s = step0; s < step0 + n_steps; ++s) {
        for (int64_t v = 0; v < n_virtual; ++v) {
            const int32_t k = orc_poisson_count_stream((uint32_t)v, (uint64_t)s, stream, seed, thr + 4 * v);
            for (int32_t j = 0; j < k; ++j) {
                if (n < cap) {
                    emit_step[n] = s;
                    source[n] = (int32_t)v;
                }
                ++n;
            }
        }
    }
    return n;
}

int64_t orc_poisson_fill(int64_t n_virtual, const uint32_t* thr, uint64_t seed, int64_t step0, int64_t n_steps,
                         int64_t cap, int64_t* emit_step, int32_t* source)
{
    int64_t n = 0;
    for (int64_t s = step0; s < step0 + n_steps; ++s) {
        for (int64_t v = 0; v < n_virtual; ++v) {
            const int32_t k = orc_poisson_count((uint32_t)v, (uint64_t)s, seed, thr + 4 * v);
            for (int32_t j = 0; j < k; ++j) {
                if (n < cap) {
                    emit_step[n] = s;
                    source[n] = (int32_t)v;
                }
                ++n;
            }
        }
    }
    return n;
}

/* CSR by source with a stable counting sort (rows keep edge-list order). Used where the
 * canonical in-row order does not matter (timed CPU baseline on tens of millions of edges);
 * the lexsort construction in glif_oracle.py is the one the device CSR is compared with. */
void orc_csr_by_source(int64_t n_rows, int64_t n_edges, const uint32_t* src, const uint32_t* trg,
                       const float* weight, const uint16_t* delay, const uint8_t* port, int64_t* rowptr,
                       int32_t* o_trg, int32_t* o_port, int32_t* o_delay, double* o_weight)
{
    for (int64_t r = 0; r <= n_rows; ++r) rowptr[r] = 0;
    for (int64_t k = 0; k < n_edges; ++k) ++rowptr[src[k] + 1];
    for (int64_t r = 0; r < n_rows; ++r) rowptr[r + 1] += rowptr[r];
    int64_t* fill = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n_rows > 0 ? n_rows : 1));
    if (!fill) return;
    memcpy(fill, rowptr, sizeof(int64_t) * (size_t)n_rows);
    for (int64_t k = 0; k < n_edges; ++k) {
        const int64_t pos = fill[src[k]]++;
        o_trg[pos] = (int32_t)trg[k];
        o_port[pos] = port[k];
        o_delay[pos] = delay[k];
        o_weight[pos] = (double)weight[k];
    }
    free(fill);
}

/* ---- CPU restatement of the device-side network generator (bmtk_b200/csrc/generate.cu): candidate k of target t
 * owns the Philox counters (t, k, 0, 0) and (t, k, 1, 0); every floating-point step is one IEEE single-precision
 * operation in the order written here (fmaf where the device fuses), so the edge list is identical bit for bit.
 * The reference has no counterpart (bmtk.builder evaluates Python connection rules per node pair,
 * examples/point_450glifs/build_network.py); this is the checker of the synthetic stand-in. */
typedef struct {
    uint32_t n_neurons, n_types, lo, hi;
    const uint16_t* type_index;
    const uint8_t* type_is_inh;
    const float *x, *y;
    const float* sigma;
    const float* w_base;
    const float *q_exc, *q_inh;
    const float* lambda;
    const float *gauss_table, *lognorm_table;
    const uint32_t* cell_start[2];
    const uint32_t* cell_count[2];
    const uint32_t* cell_ids[2];
    uint32_t class_size[2];
    float cell_max[2];
    uint32_t grid;
    float radius, inv_cell, inh_scale, delay_min_ms, delay_max_ms, dt;
    uint64_t seed;
} orc_gen_spec;

static float gen_u24(uint32_t r) { return (float)(r >> 8) * 5.9604644775390625e-08f; }

int64_t orc_generate_distance_edges(const orc_gen_spec* g, int64_t cap, uint32_t* src, uint32_t* trg, float* weight,
                                    uint16_t* delay, uint8_t* port)
{
    const uint32_t key[2] = { (uint32_t)g->seed, (uint32_t)(g->seed >> 32) };
    int64_t n = 0;
    for (uint32_t t = g->lo; t < g->hi; ++t) {
        const uint32_t tt = g->type_index[t];
        const float lam = g->lambda[tt];
        const uint32_t base = (uint32_t)lam;
        uint32_t r[4];
        const uint32_t c0[4] = { t, 0xffffffffu, 2u, 0u };
        orc_philox4x32_10(c0, key, r);
        const uint32_t K = base + (gen_u24(r[0]) < lam - (float)base ? 1u : 0u);
        for (uint32_t k = 0; k < K; ++k) {
            uint32_t a[4], b[4];
            const uint32_t ca[4] = { t, k, 0u, 0u }, cb[4] = { t, k, 1u, 0u };
            orc_philox4x32_10(ca, key, a);
            orc_philox4x32_10(cb, key, b);
            const float qe = g->q_exc[tt], qi = g->q_inh[tt];
            const uint32_t sc = gen_u24(a[0]) * (qe + qi) >= qe ? 1u : 0u;
            const float sg = g->sigma[sc * g->n_types + tt];
            const float px = fmaf(g->gauss_table[a[1] >> 20], sg, g->x[t]);
            const float py = fmaf(g->gauss_table[a[2] >> 20], sg, g->y[t]);
            const float R = g->radius;
            if (!(fmaf(px, px, py * py) < R * R)) continue;
            const int cx = (int)floorf((px + R) * g->inv_cell), cy = (int)floorf((py + R) * g->inv_cell);
            if (cx < 0 || cy < 0 || cx >= (int)g->grid || cy >= (int)g->grid) continue;
            const uint32_t cell = (uint32_t)cx * g->grid + (uint32_t)cy;
            const uint32_t cn = g->cell_count[sc][cell];
            if (!(gen_u24(a[3]) * g->cell_max[sc] < (float)cn)) continue;
            uint32_t pick = (uint32_t)(gen_u24(b[0]) * (float)cn);
            if (pick >= cn) pick = cn - 1u;
            const uint32_t s = g->cell_ids[sc][g->cell_start[sc][cell] + pick];
            if (s == t) continue;
            const uint32_t st = g->type_index[s];
            float w = g->w_base[st * g->n_types + tt] * g->lognorm_table[b[1] >> 20];
            const int s_inh = g->type_is_inh[st] != 0, t_inh = g->type_is_inh[tt] != 0;
            if (s_inh) w = w * -g->inh_scale;
            const float d_ms = fmaf(gen_u24(b[2]), g->delay_max_ms - g->delay_min_ms, g->delay_min_ms);
            const float d_steps = rintf(d_ms / g->dt);
            if (n < cap) {
                src[n] = s; trg[n] = t; weight[n] = w;
                delay[n] = (uint16_t)(d_steps < 1.f ? 1.f : d_steps);
                port[n] = (uint8_t)(s_inh + 2 * t_inh);
            }
            ++n;
        }
    }
    return n;
}

/* ============================================================================================
 * Single-precision restatement of the engine's stepping with DETERMINISTIC delivery.
 *
 * The fp64 functions above state the model; this one states the engine's own arithmetic contract, so that the
 * CUDA path can be compared bit for bit instead of within a tolerance:
 *   - per-type constants are the fp64 values of orc_glif_consts_init rounded to float (a type without after-spike
 *     currents gets decay 1 / coefficient 0, an unused receptor port all zeros);
 *   - one neuron step is the sequence of single IEEE-754 operations written in step_f32 (fmaf where a fused
 *     multiply-add is meant; the file is compiled with -ffp-contract=off, so nothing else fuses);
 *   - spikes are delivered once per exchange window of `window` steps (windows restart at every chunk of
 *     `chunk_steps` steps, as the engine's run loop cuts them): the window's spikes - neurons, replayed virtual
 *     spikes, Poisson cells - are ordered by (emitting step, source id), every spike's row is walked in CSR order
 *     (delay, port, target; ties in edge-list order), the weights that meet in one ring cell are added left to
 *     right in that order starting from the first, and the cell receives that sum with one addition.
 * What NEST does inside nest.Simulate (bmtk/simulator/pointnet/pointsimulator.py:166) is fp64; the fp64 oracle
 * is the reference for results, this restatement pins the device arithmetic. */
typedef struct {
    float P11[ORC_MAX_PORTS], P21[ORC_MAX_PORTS], P31[ORC_MAX_PORTS], P32[ORC_MAX_PORTS], psc_init[ORC_MAX_PORTS];
    float asc_decay[2], asc_coeff[2], asc_refr[2], asc_amps[2], asc_rec[2];
    float P33, P30, th_inf, i_e, v_reset, E_L, inv_G, delta_gain;
    float theta_spike_decay, theta_spike_refr, th_spike_add, reset_fraction, reset_add, phi, abpara, theta_voltage_decay;
    int32_t n_ref, sdt, adapt, iaf;
} orc_f32_consts;

static void f32_consts_init(const orc_glif_params* p, double h, orc_f32_consts* f)
{
    orc_glif_consts c;
    orc_glif_consts_init(p, h, &c);
    memset(f, 0, sizeof(*f));
    for (int k = 0; k < c.n_ports; ++k) {
        f->P11[k] = (float)c.P11[k]; f->P21[k] = (float)c.P21[k]; f->P31[k] = (float)c.P31[k];
        f->P32[k] = (float)c.P32[k]; f->psc_init[k] = (float)c.psc_init[k];
    }
    for (int j = 0; j < 2; ++j) {
        if (c.has_asc) {
            f->asc_decay[j] = (float)c.asc_decay_rate[j]; f->asc_coeff[j] = (float)c.asc_stable_coeff[j];
            f->asc_refr[j] = (float)c.asc_refr_rate[j]; f->asc_amps[j] = (float)c.asc_amps[j];
            f->asc_rec[j] = (float)(c.asc_stable_coeff[j] / c.asc_decay_rate[j]);
        } else {
            f->asc_decay[j] = 1.f; f->asc_refr[j] = 1.f;
        }
    }
    f->P33 = (float)c.P33; f->P30 = (float)c.P30; f->th_inf = (float)c.th_inf; f->i_e = (float)c.I_e;
    f->v_reset = (float)c.v_reset; f->E_L = (float)c.E_L; f->inv_G = (float)(1.0 / c.G); f->delta_gain = c.delta ? 1.f : 0.f;
    f->theta_spike_decay = (float)c.theta_spike_decay; f->theta_spike_refr = (float)c.theta_spike_refr_decay;
    f->th_spike_add = (float)c.th_spike_add; f->reset_fraction = (float)c.reset_fraction; f->reset_add = (float)c.reset_add;
    f->phi = (float)c.phi; f->abpara = (float)c.abpara; f->theta_voltage_decay = (float)c.theta_voltage_decay;
    f->n_ref = c.n_ref; f->sdt = c.has_theta_spike; f->adapt = c.has_theta_voltage; f->iaf = c.iaf;
}

typedef struct {
    int64_t n_neurons, n_virtual;
    const int32_t* type_index;
    int32_t n_types;
    const orc_glif_params* types;
    const int64_t* rowptr;
    const int32_t *target, *port, *delay;
    const float* weight;
    int32_t max_delay, window, theta_any;   /* theta_any: some type has threshold dynamics (the device then adds the
                                               two components to th_inf for every type) */
    int64_t chunk_steps;
    const int64_t* in_step_ptr;             /* replayed virtual spikes by emitting step, [step0 + n_steps + 1] */
    const int32_t* in_src;
    const float* poisson_rate_hz;           /* on-line Poisson cells (NULL = none) */
    uint64_t poisson_seed;
    uint32_t poisson_stream;
    int64_t n_clamp;
    const int64_t* ce_step;
    const int32_t* ce_target;
    const float* ce_delta;
    double dt;
    int64_t step0, n_steps;
    float *U, *asc0, *asc1, *y1, *y2, *th_spike, *th_voltage, *i_ext, *ring;   /* ring: (max_delay + window) slots */
    int32_t* refr;
    int64_t spike_cap;
    int64_t* n_spikes;
    int64_t* spike_step;
    int32_t* spike_id;
    int32_t n_probe;
    const int32_t* probe_ids;
    int32_t probe_interval, n_probe_vars;
    uint32_t probe_vars;
    float* trace;
    int64_t* n_samples;
    int64_t* n_events;
} orc_f32_args;

void orc_f32_init_state(const orc_f32_args* a)
{
    const int64_t N = a->n_neurons, S = (int64_t)a->max_delay + a->window;
    for (int64_t i = 0; i < N; ++i) {
        const orc_glif_params* p = &a->types[a->type_index[i]];
        a->U[i] = (float)(p->V_m - p->E_L);
        a->asc0[i] = (float)p->asc_init[0];
        a->asc1[i] = (float)p->asc_init[1];
        a->th_spike[i] = a->th_voltage[i] = a->i_ext[i] = 0.f;
        a->refr[i] = 0;
    }
    memset(a->y1, 0, sizeof(float) * ORC_MAX_PORTS * N);
    memset(a->y2, 0, sizeof(float) * ORC_MAX_PORTS * N);
    memset(a->ring, 0, sizeof(float) * S * ORC_MAX_PORTS * N);
}

typedef struct { uint64_t key; } f32_item;   /* emitting step << 32 | source id */
static int f32_item_cmp(const void* x, const void* y)
{
    const uint64_t a = ((const f32_item*)x)->key, b = ((const f32_item*)y)->key;
    return a < b ? -1 : a > b;
}

int orc_f32_run(orc_f32_args* a)
{
    const int64_t N = a->n_neurons, S = (int64_t)a->max_delay + a->window;
    const double h = a->dt;
    orc_f32_consts* C = (orc_f32_consts*)malloc(sizeof(orc_f32_consts) * (size_t)a->n_types);
    float* acc = (float*)malloc(sizeof(float) * (size_t)(S * ORC_MAX_PORTS * N));
    uint8_t* seen = (uint8_t*)calloc((size_t)(S * ORC_MAX_PORTS * N), 1);
    int64_t* touched = NULL;
    int64_t touched_cap = 0, n_touched = 0;
    f32_item* items = NULL;
    int64_t item_cap = 0, n_items = 0;
    uint32_t* thr = NULL;
    if (!C || !acc || !seen) return -1;
    for (int t = 0; t < a->n_types; ++t) f32_consts_init(&a->types[t], h, &C[t]);
    if (a->poisson_rate_hz) {
        thr = (uint32_t*)malloc(sizeof(uint32_t) * 4 * (size_t)a->n_virtual);
        for (int64_t v = 0; v < a->n_virtual; ++v) orc_poisson_thresholds((double)a->poisson_rate_hz[v] * h * 1e-3, &thr[4 * v]);
    }
    int64_t ce = 0;
    while (ce < a->n_clamp && a->ce_step[ce] < a->step0) ++ce;
    int status = 0;
#define F32_PUSH(step_, src_) do { \
        if (n_items == item_cap) { item_cap = item_cap ? 2 * item_cap : 4096; items = (f32_item*)realloc(items, sizeof(f32_item) * (size_t)item_cap); } \
        items[n_items++].key = ((uint64_t)(step_) << 32) | (uint64_t)(src_); } while (0)
    int64_t n = a->step0;
    const int64_t end = a->step0 + a->n_steps;
    while (n < end) {
        int64_t chunk = end - n < a->chunk_steps ? end - n : a->chunk_steps;
        const int64_t chunk_end = n + chunk;
        while (n < chunk_end) {
            const int64_t w = chunk_end - n < a->window ? chunk_end - n : a->window;
            n_items = 0;
            for (int64_t s = 0; s < w; ++s, ++n) {
                while (ce < a->n_clamp && a->ce_step[ce] <= n) {
                    a->i_ext[a->ce_target[ce]] = a->i_ext[a->ce_target[ce]] + a->ce_delta[ce];
                    ++ce;
                }
                const int64_t slot = n % S;
                for (int64_t i = 0; i < N; ++i) {
                    const orc_f32_consts* c = &C[a->type_index[i]];
                    float in[ORC_MAX_PORTS];
                    for (int p = 0; p < ORC_MAX_PORTS; ++p) {
                        float* cell = &a->ring[(slot * ORC_MAX_PORTS + p) * N + i];
                        in[p] = *cell;
                        *cell = 0.f;
                    }
                    const float v_old = a->U[i];
                    const int refr = a->refr[i] > 0;
                    const int rf_dec = a->refr[i] - 1;
                    const int ends = refr && rf_dec == 0;
                    /* integrating branch (evaluated for every neuron, selected below, as on the device) */
                    const float asc_sum = fmaf(c->asc_coeff[0], a->asc0[i], c->asc_coeff[1] * a->asc1[i]);
                    const float drive = (a->i_ext[i] + c->i_e) + asc_sum;
                    float u = fmaf(v_old, c->P33, drive * c->P30);
                    for (int p = 0; p < ORC_MAX_PORTS; ++p)
                        u = u + fmaf(c->P31[p], a->y1[p * N + i], c->P32[p] * a->y2[p * N + i]);
                    u = fmaf(c->delta_gain, (in[0] + in[1]) + (in[2] + in[3]), u);
                    float th = c->th_inf;
                    float ths_int = a->th_spike[i], thv_int = a->th_voltage[i];
                    if (a->theta_any) {
                        if (c->sdt) ths_int = a->th_spike[i] * c->theta_spike_decay;
                        if (c->adapt) {
                            const float beta = drive * c->inv_G;
                            const float d = c->phi * (v_old - beta);
                            const float ab = c->abpara * beta;
                            const float rest = (a->th_voltage[i] - d) - ab;
                            thv_int = fmaf(c->theta_voltage_decay, rest, d * c->P33) + ab;
                        }
                        th = th + (ths_int + thv_int);
                    }
                    const int fire = !refr && (c->iaf ? (u >= th) : (u > th));
                    if (c->iaf && fire) u = c->v_reset;
                    const float u_end = c->sdt ? fmaf(c->reset_fraction, v_old, c->reset_add) : c->v_reset;
                    a->U[i] = refr ? (ends ? u_end : v_old) : u;
                    a->asc0[i] = refr ? (ends ? fmaf(a->asc0[i], c->asc_refr[0], c->asc_amps[0]) : a->asc0[i]) : a->asc0[i] * c->asc_decay[0];
                    a->asc1[i] = refr ? (ends ? fmaf(a->asc1[i], c->asc_refr[1], c->asc_amps[1]) : a->asc1[i]) : a->asc1[i] * c->asc_decay[1];
                    if (a->theta_any) {
                        a->th_spike[i] = refr ? ((ends && c->sdt) ? fmaf(a->th_spike[i], c->theta_spike_refr, c->th_spike_add) : a->th_spike[i]) : ths_int;
                        a->th_voltage[i] = refr ? a->th_voltage[i] : thv_int;
                    }
                    a->refr[i] = refr ? rf_dec : (fire ? c->n_ref : a->refr[i]);
                    for (int p = 0; p < ORC_MAX_PORTS; ++p) {
                        const float y1o = a->y1[p * N + i];
                        a->y2[p * N + i] = fmaf(c->P21[p], y1o, c->P11[p] * a->y2[p * N + i]);
                        a->y1[p * N + i] = fmaf(c->P11[p], y1o, c->psc_init[p] * in[p]);
                    }
                    if (fire) {
                        if (a->spike_step) {
                            if (*a->n_spikes < a->spike_cap) {
                                a->spike_step[*a->n_spikes] = n + 1;
                                a->spike_id[*a->n_spikes] = (int32_t)i;
                            } else {
                                status = 1;
                            }
                        }
                        ++*a->n_spikes;
                        F32_PUSH(n, i);
                    }
                }
                if (a->in_step_ptr)
                    for (int64_t k = a->in_step_ptr[n]; k < a->in_step_ptr[n + 1]; ++k) F32_PUSH(n, N + a->in_src[k]);
                if (thr)
                    for (int64_t v = 0; v < a->n_virtual; ++v) {
                        const int32_t cnt = orc_poisson_count_stream((uint32_t)v, (uint64_t)n, a->poisson_stream, a->poisson_seed, &thr[4 * v]);
                        for (int32_t q = 0; q < cnt; ++q) F32_PUSH(n, N + v);
                    }
                if (a->n_probe > 0 && (n + 1) % a->probe_interval == 0) {
                    const int nv = a->n_probe_vars > 0 ? a->n_probe_vars : 1;
                    float* row = a->trace + (*a->n_samples) * a->n_probe * nv;
                    for (int v = 0; v < nv; ++v) {
                        const uint32_t code = a->n_probe_vars > 0 ? (a->probe_vars >> (4 * v)) & 15u : 0u;
                        for (int q = 0; q < a->n_probe; ++q) {
                            const int32_t i = a->probe_ids[q];
                            const orc_f32_consts* c = &C[a->type_index[i]];
                            float x;
                            switch (code) {
                                case 1: x = ((a->y2[i] + a->y2[N + i]) + a->y2[2 * N + i]) + a->y2[3 * N + i]; break;
                                case 2: x = fmaf(c->asc_rec[0], a->asc0[i], c->asc_rec[1] * a->asc1[i]); break;
                                case 3: x = ((c->th_inf + a->th_spike[i]) + a->th_voltage[i]) + c->E_L; break;
                                case 4: x = a->th_spike[i]; break;
                                case 5: x = a->th_voltage[i]; break;
                                case 6: x = a->i_ext[i] + c->i_e; break;
                                default: x = a->U[i] + c->E_L;
                            }
                            row[v * a->n_probe + q] = x;
                        }
                    }
                    ++*a->n_samples;
                }
            }
            /* ---- the window's delivery */
            qsort(items, (size_t)n_items, sizeof(f32_item), f32_item_cmp);
            n_touched = 0;
            for (int64_t it = 0; it < n_items; ++it) {
                const int64_t step = (int64_t)(items[it].key >> 32), src = (int64_t)(items[it].key & 0xffffffffu);
                for (int64_t k = a->rowptr[src]; k < a->rowptr[src + 1]; ++k) {
                    const int64_t cell = (((step + a->delay[k]) % S) * ORC_MAX_PORTS + a->port[k]) * N + a->target[k];
                    if (!seen[cell]) {
                        seen[cell] = 1;
                        acc[cell] = a->weight[k];
                        if (n_touched == touched_cap) {
                            touched_cap = touched_cap ? 2 * touched_cap : 4096;
                            touched = (int64_t*)realloc(touched, sizeof(int64_t) * (size_t)touched_cap);
                        }
                        touched[n_touched++] = cell;
                    } else {
                        acc[cell] = acc[cell] + a->weight[k];
                    }
                }
                *a->n_events += a->rowptr[src + 1] - a->rowptr[src];
            }
            for (int64_t k = 0; k < n_touched; ++k) {
                a->ring[touched[k]] = a->ring[touched[k]] + acc[touched[k]];
                seen[touched[k]] = 0;
            }
        }
    }
#undef F32_PUSH
    free(C); free(acc); free(seen); free(touched); free(items); free(thr);
    return status;
}
