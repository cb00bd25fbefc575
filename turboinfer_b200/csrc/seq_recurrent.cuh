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

enum { LIN_GATES_GIVEN = 0, LIN_GATES_GLA = 1, LIN_GATES_HGRN2 = 2 };
// What the scan does to its raw operands while it stages them (fp32):
//   GIVEN  q and the decay are used as they are
//   GLA    decay = exp(log_sigmoid(z + bias) / tau), log_sigmoid(x) = min(x, 0) - log1p(exp(-|x|))
//   HGRN2  q = z_q * sigmoid(z_q), decay = lower + (1 - lower) * sigmoid(z + bias)
__device__ __forceinline__ void lin_gates(int mode, float& q, float& dec, float bias, float lower, float inv_tau) {
    if (mode == LIN_GATES_GLA) {
        const float x = dec + bias;
        dec = expf((fminf(x, 0.f) - log1pf(expf(-fabsf(x)))) * inv_tau);
    } else if (mode == LIN_GATES_HGRN2) {
        q = q / (1.f + expf(-q));
        dec = lower + (1.f - lower) / (1.f + expf(-(dec + bias)));
    }
}

struct LinScanArgs {
    const float *q, *k, *a, *v;   // rows t, head hd: q / k / a at [t * ld + hd * dk + i], v at [t * ldv + hd * dv + j]; k == null: w = 1 - a
    int ldq, ldk, lda, ldv;
    int gates;                    // LIN_GATES_*: how q and a become the query and the decay
    const float *bias, *lower;    // [heads * dk] each (lower: HGRN2 only)
    float inv_tau;
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
            float dec = a.a[t * a.lda + (size_t)hd * dk + i], qv = a.q[t * a.ldq + (size_t)hd * dk + i];
            if (a.gates != LIN_GATES_GIVEN) lin_gates(a.gates, qv, dec, a.bias[hd * dk + i], a.lower ? a.lower[hd * dk + i] : 0.f, a.inv_tau);
            stage[(c * 3 + 0) * dk + i] = qv * a.qscale;
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
// Key channels of 32 / 64 / 128: a BLOCK owns 32 value columns of a head (grid z = column group) and its NW warps split the key
// channels, so a lane keeps DK / NW entries of its state column in registers and a token costs DK / NW dependent multiply-adds a
// lane instead of DK.  Tokens are taken CH at a time: the chunk's q, w, a vectors and v columns go to shared memory while the
// NEXT chunk's operands are already requested; every warp runs the chunk's tokens over its channels and leaves a partial
// output per token; the NW partials are summed in warp order (the result does not depend on timing).  The organisation of the
// wkv scan of seq_kernels.cuh, with the output read after the update and value columns that need not be as many as key channels.
template <int DK, int CH, int NW>
__global__ void __launch_bounds__(32 * NW) linear_scan_split_kernel(LinScanArgs a, StepMeta m) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    constexpr int RP = DK / NW, NT = 32 * NW, PER = CH * DK / NT, VPER = (CH * 32 + NT - 1) / NT;
    static_assert(DK % NW == 0 && RP % 4 == 0 && (CH * DK) % NT == 0, "chunk staging must divide evenly");
    __shared__ __align__(16) float buf[CH][3][DK];
    __shared__ float vbuf[CH][32];
    __shared__ float part[NW][CH][32];
    const int e = blockIdx.x, hd = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dv = a.dv, col0 = blockIdx.z * 32, j = col0 + lane;
    const bool own = j < dv;
    float* Sg = a.state + ((size_t)m.ent_slot[e] * a.heads + hd) * (size_t)DK * dv;
    const bool fresh = (m.ent_pos0[e] == 0);
    float S[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) S[i] = (own && !fresh) ? Sg[(size_t)(warp * RP + i) * dv + j] : 0.f;
    const int t0 = m.ent_row0[e], t1 = m.ent_row0[e + 1];
    float gb[PER], gl[PER];   // the gates' per-channel constants of the channels this thread stages
#pragma unroll
    for (int p = 0; p < PER; ++p) {
        const int i = (tid + NT * p) % DK;
        gb[p] = a.gates != LIN_GATES_GIVEN ? a.bias[hd * DK + i] : 0.f;
        gl[p] = a.lower ? a.lower[hd * DK + i] : 0.f;
    }
    float nq[PER], nk[PER], na[PER], nv[VPER];
    auto fetch = [&](int tc) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int x = tid + NT * p, c = x / DK, i = x % DK;
            const size_t t = (size_t)min(tc + c, t1 - 1);
            nq[p] = a.q[t * a.ldq + (size_t)hd * DK + i];
            na[p] = a.a[t * a.lda + (size_t)hd * DK + i];
            nk[p] = a.k ? a.k[t * a.ldk + (size_t)hd * DK + i] : 0.f;
        }
#pragma unroll
        for (int p = 0; p < VPER; ++p) {
            const int x = tid + NT * p, c = x >> 5, l = x & 31;
            nv[p] = (c < CH && col0 + l < dv) ? a.v[(size_t)min(tc + c, t1 - 1) * a.ldv + (size_t)hd * dv + col0 + l] : 0.f;
        }
    };
    auto emit = [&](int tc) {   // out[t][j] = sum over the warps' partials, chunk starting at row tc
        for (int x = tid; x < CH * 32; x += NT) {
            const int c = x >> 5, l = x & 31;
            if (tc + c < t1 && col0 + l < dv) {
                float s = part[0][c][l];
#pragma unroll
                for (int w = 1; w < NW; ++w) s += part[w][c][l];
                a.out[(size_t)(tc + c) * (a.heads * dv) + (size_t)hd * dv + col0 + l] = s;
            }
        }
    };
    fetch(t0);
    for (int tc = t0; tc < t1; tc += CH) {
        if (tc > t0) emit(tc - CH);
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int x = tid + NT * p, c = x / DK, i = x % DK;
            float qv = nq[p], dec = na[p];
            if (a.gates != LIN_GATES_GIVEN) lin_gates(a.gates, qv, dec, gb[p], gl[p], a.inv_tau);
            buf[c][0][i] = qv * a.qscale;
            buf[c][1][i] = a.k ? nk[p] : 1.f - dec;
            buf[c][2][i] = dec;
        }
#pragma unroll
        for (int p = 0; p < VPER; ++p) {
            const int x = tid + NT * p;
            if (x < CH * 32) vbuf[x >> 5][x & 31] = nv[p];
        }
        __syncthreads();
        if (tc + CH < t1) fetch(tc + CH);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (tc + c < t1) {
                float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
                const float v = vbuf[c][lane];
#pragma unroll
                for (int i = 0; i < RP; i += 4) {
                    const int ch = warp * RP + i;
                    const float4 q4 = *reinterpret_cast<const float4*>(&buf[c][0][ch]);
                    const float4 w4 = *reinterpret_cast<const float4*>(&buf[c][1][ch]);
                    const float4 a4 = *reinterpret_cast<const float4*>(&buf[c][2][ch]);
                    S[i] = fmaf(a4.x, S[i], w4.x * v);
                    acc0 = fmaf(q4.x, S[i], acc0);
                    S[i + 1] = fmaf(a4.y, S[i + 1], w4.y * v);
                    acc1 = fmaf(q4.y, S[i + 1], acc1);
                    S[i + 2] = fmaf(a4.z, S[i + 2], w4.z * v);
                    acc2 = fmaf(q4.z, S[i + 2], acc2);
                    S[i + 3] = fmaf(a4.w, S[i + 3], w4.w * v);
                    acc3 = fmaf(q4.w, S[i + 3], acc3);
                }
                part[warp][c][lane] = (acc0 + acc1) + (acc2 + acc3);
            }
        }
        __syncthreads();
    }
    emit(t0 + (t1 - t0 - 1) / CH * CH);
    if (own) {
#pragma unroll
        for (int i = 0; i < RP; ++i) Sg[(size_t)(warp * RP + i) * dv + j] = S[i];
    }
}

inline size_t linear_scan_smem_bytes(int dk, int threads, bool state_in_smem) {
    return sizeof(float) * ((size_t)kLinScanChunk * (3 * dk + threads) + (state_in_smem ? (size_t)dk * threads : 0));
}

}  // namespace seq
}  // namespace tib
