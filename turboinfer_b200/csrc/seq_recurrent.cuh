// seq_recurrent.cuh -- gated linear recurrences of the layered sequence engine, beside the token-shifted wkv recurrence of
// seq_kernels.cuh:
//
//     S_t = diag(a_t) S_(t-1) + w_t v_t^T        S: [dk key channels][dv value channels] per head, fp32, one per live sequence
//     o_t = S_t^T (qscale * q_t)                 (the output reads the state AFTER the token was written)
//
// with a per-key-channel decay a_t in (0, 1).  Two mixers use it:
//   gla    w = k,     a = sigmoid(z + b)^(1 / tau)          (z from a two-matrix projection)
//   hgrn2  w = 1 - a, a = l + (1 - l) sigmoid(z + b)        (the forget gate also decides what is written; q = silu(.))
// The decays, their logarithms and exponentials, the state and the sums are fp32 in both compute modes.  Operands are slices of
// the mixer's fused input projection, so every pointer comes with its own row stride.
#pragma once
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

// z [T][C] -> decay = exp(log_sigmoid(z + bias) / tau), in place; log_sigmoid(x) = min(x, 0) - log1p(exp(-|x|))
__global__ void gla_decay_kernel(float* z, const float* bias, float inv_tau, int C, size_t n) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float x = z[i] + bias[i % C];
        const float ls = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
        z[i] = expf(ls * inv_tau);
    }
}
// in the fused projection rows: q <- silu(q), f <- lower + (1 - lower) * sigmoid(f + bias); C = heads * dk coordinates each
__global__ void hgrn2_gates_kernel(float* proj, int ld, int off_q, int off_f, const float* bias, const float* lower, int C, int T) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const size_t n = (size_t)T * C;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / C, c = i % C;
        float* row = proj + t * ld;
        const float q = row[off_q + c];
        row[off_q + c] = q / (1.f + expf(-q));
        const float lo = lower[c];
        row[off_f + c] = lo + (1.f - lo) / (1.f + expf(-(row[off_f + c] + bias[c])));
    }
}

struct LinScanArgs {
    const float *q, *k, *a, *v;   // rows t, head hd: q / k / a at [t * ld + hd * dk + i], v at [t * ldv + hd * dv + j]; k == null: w = 1 - a
    int ldq, ldk, lda, ldv;
    float qscale;
    float* state;                 // [slots][heads][dk][dv]
    float* out;                   // [T][heads * dv]
    int heads, dk, dv;
};

// One block per (entry, head, group of value columns): thread j owns column j of S.  DKR > 0: the column lives in registers
// (dk <= DKR, the loop bound is uniform); DKR = 0: in shared memory, any dk.  Tokens are staged CH at a time (q, w, a of the
// chunk and the block's v columns in shared memory) so that the serial loop over tokens only touches shared memory.
constexpr int kLinScanChunk = 8;
template <int DKR>
__global__ void __launch_bounds__(128) linear_scan_kernel(LinScanArgs a, StepMeta m) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    extern __shared__ float lsm[];   // [CH][3][dk], [CH][blockDim.x] values, then (DKR == 0) S [dk][blockDim.x]
    constexpr int CH = kLinScanChunk;
    const int e = blockIdx.x, hd = blockIdx.y, dk = a.dk, dv = a.dv;
    const int j = blockIdx.z * blockDim.x + threadIdx.x;
    const bool own = j < dv;
    float* stage = lsm;
    float* vst = lsm + (size_t)CH * 3 * dk;
    float* Ssm = vst + (size_t)CH * blockDim.x;
    float* Sg = a.state + ((size_t)m.ent_slot[e] * a.heads + hd) * (size_t)dk * dv;
    const bool fresh = (m.ent_pos0[e] == 0);
    float S[DKR > 0 ? DKR : 1];
    if (DKR > 0) {
#pragma unroll
        for (int i = 0; i < DKR; ++i) S[i] = (own && !fresh && i < dk) ? Sg[(size_t)i * dv + j] : 0.f;
    } else {
        for (int i = 0; i < dk; ++i) Ssm[(size_t)i * blockDim.x + threadIdx.x] = (own && !fresh) ? Sg[(size_t)i * dv + j] : 0.f;
    }
    const int t0 = m.ent_row0[e], t1 = m.ent_row0[e + 1];
    for (int tc = t0; tc < t1; tc += CH) {
        const int nc = min(CH, t1 - tc);
        __syncthreads();
        for (int x = threadIdx.x; x < nc * dk; x += blockDim.x) {
            const int c = x / dk, i = x % dk;
            const size_t t = (size_t)(tc + c);
            const float dec = a.a[t * a.lda + (size_t)hd * dk + i];
            stage[(c * 3 + 0) * dk + i] = a.q[t * a.ldq + (size_t)hd * dk + i] * a.qscale;
            stage[(c * 3 + 1) * dk + i] = a.k ? a.k[t * a.ldk + (size_t)hd * dk + i] : 1.f - dec;
            stage[(c * 3 + 2) * dk + i] = dec;
        }
        for (int c = 0; c < nc; ++c) vst[c * blockDim.x + threadIdx.x] = own ? a.v[(size_t)(tc + c) * a.ldv + (size_t)hd * dv + j] : 0.f;
        __syncthreads();
#pragma unroll 1
        for (int c = 0; c < nc; ++c) {
            {
                const float* qs = stage + (c * 3 + 0) * dk;
                const float* ws = stage + (c * 3 + 1) * dk;
                const float* as = stage + (c * 3 + 2) * dk;
                const float v = vst[c * blockDim.x + threadIdx.x];
                float acc0 = 0.f, acc1 = 0.f;
                if (DKR > 0) {
#pragma unroll
                    for (int i = 0; i < DKR; i += 2) {
                        if (i < dk) {
                            S[i] = fmaf(as[i], S[i], ws[i] * v);
                            acc0 = fmaf(qs[i], S[i], acc0);
                        }
                        if (i + 1 < dk) {
                            S[i + 1] = fmaf(as[i + 1], S[i + 1], ws[i + 1] * v);
                            acc1 = fmaf(qs[i + 1], S[i + 1], acc1);
                        }
                    }
                } else {
                    for (int i = 0; i < dk; ++i) {
                        float* sp = Ssm + (size_t)i * blockDim.x + threadIdx.x;
                        const float sv = fmaf(as[i], *sp, ws[i] * v);
                        *sp = sv;
                        acc0 = fmaf(qs[i], sv, acc0);
                    }
                }
                if (own) a.out[(size_t)(tc + c) * (a.heads * dv) + (size_t)hd * dv + j] = acc0 + acc1;
            }
        }
    }
    if (own) {
        if (DKR > 0) {
#pragma unroll
            for (int i = 0; i < DKR; ++i)
                if (i < dk) Sg[(size_t)i * dv + j] = S[i];
        } else {
            for (int i = 0; i < dk; ++i) Sg[(size_t)i * dv + j] = Ssm[(size_t)i * blockDim.x + threadIdx.x];
        }
    }
}
inline size_t linear_scan_smem_bytes(int dk, int threads, bool state_in_smem) {
    return sizeof(float) * ((size_t)kLinScanChunk * (3 * dk + threads) + (state_in_smem ? (size_t)dk * threads : 0));
}

}  // namespace seq
}  // namespace tib
