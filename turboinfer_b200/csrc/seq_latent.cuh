// seq_latent.cuh -- latent attention of the layered sequence engine: softmax attention whose per-head keys and values are
// linear images (Uk, Uv) of ONE cached low-rank vector c per token, plus one rotated key part shared by all heads.
//
// The cache holds, per token, the row [c (rank) | rotated key part (rot)] in fp32 -- nothing per head.  The per-head products
// are moved to the query side and behind the weighted sum, which is the same arithmetic re-associated:
//     score_h(i, j) = (q_h . Uk_h c_j + qr_h . kr_j) * scale = ((Uk_h^T q_h) . c_j + qr_h . kr_j) * scale
//     out_h(i)      = sum_j p_h(i, j) Uv_h c_j                = Uv_h (sum_j p_h(i, j) c_j)
// so the attention itself is one key/value head of size rank + rot (values = the first rank coordinates of the key row) shared
// by all query heads, and runs on the paged attention kernels of seq_kernels.cuh / seq_attn_tc.cuh (window 0, value pool = key
// pool, sink term).  This file holds what is special: the cache append and the query's rotated part.
#pragma once
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

struct LatentShape {
    int heads, dim, rot, rank;   // per head: `dim` unrotated and `rot` rotated query coordinates; cached row = rank + rot
    int ld;                      // row stride of the fused projection [q | dkv | ...]
    int off_q, off_dkv;          // column of q (heads * (dim + rot)) and of the down projection (rank + rot); off_dkv < 0: the layer
                                 // reads another layer's cache and appends nothing
    float eps;
};
// One block per row.  Own cache: c = dkv[:rank] / rms * cnorm -> page row; rotated key part -> behind it.  Every head's rotated
// query part -> qabs[t][h][rank ...] (the absorbed part [0, rank) is written by the product with Uk^T).  Pairs (2i, 2i + 1) of
// the rotated parts turn by position * inv_freq[i], angle in fp32.
__global__ void latent_prepare_kernel(const float* proj, StepMeta m, LatentShape s, const float* inv_freq, const float* cnorm, float* pool, float* qabs) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    __shared__ float red[32];
    const int t = blockIdx.x, pos = m.row_pos[t];
    const float* row = proj + (size_t)t * s.ld;
    const int kd = s.rank + s.rot;
    if (s.off_dkv >= 0) {
        const int slot = m.ent_slot[m.row_ent[t]];
        const int page = m.page_table[(size_t)slot * m.table_stride + pos / kPageTokens];
        float* dst = pool + ((size_t)page * kPageTokens + pos % kPageTokens) * kd;
        const float* src = row + s.off_dkv;
        float ss = 0.f;
        for (int i = threadIdx.x; i < s.rank; i += blockDim.x) ss += src[i] * src[i];
        ss = block_sum(ss, red);
        const float sc = 1.f / sqrtf(ss / (float)s.rank + s.eps);
        for (int i = threadIdx.x; i < s.rank; i += blockDim.x) dst[i] = src[i] * sc * cnorm[i];
        for (int i = threadIdx.x; i < s.rot / 2; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float a = src[s.rank + 2 * i], b = src[s.rank + 2 * i + 1];
            dst[s.rank + 2 * i] = a * cs - b * sn;
            dst[s.rank + 2 * i + 1] = b * cs + a * sn;
        }
    }
    for (int x = threadIdx.x; x < s.heads * (s.rot / 2); x += blockDim.x) {
        const int h = x / (s.rot / 2), i = x % (s.rot / 2);
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float* q = row + s.off_q + (size_t)h * (s.dim + s.rot) + s.dim;
        float* dst = qabs + ((size_t)t * s.heads + h) * kd + s.rank;
        const float a = q[2 * i], b = q[2 * i + 1];
        dst[2 * i] = a * cs - b * sn;
        dst[2 * i + 1] = b * cs + a * sn;
    }
}
// Uk [heads * dim][rank] -> per head its transpose [heads][rank][dim]: the weight of the query-side product
template <typename WT>
__global__ void transpose_heads_kernel(const WT* uk, int heads, int dim, int rank, WT* out) {
    const size_t n = (size_t)heads * dim * rank;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t h = i / ((size_t)dim * rank), r = (i / dim) % rank, d = i % dim;
        out[i] = uk[(h * dim + d) * rank + r];
    }
}

}  // namespace seq
}  // namespace tib
