/*
 * ti_b200_seq.h -- C ABI of libturboinfer_b200_seq.so: the layered sequence engine.
 *
 * A decoder is described layer by layer (ti_seq_layer_desc) instead of by one fixed block, and it is stepped over a RAGGED
 * batch: every step brings the next tokens of some of the live sequences -- a portion of a prompt for one, a single decoded
 * token for another -- and all of them run together.  The engine owns
 *   - a page pool for the attention layers' keys and values (64 tokens a page, one page table per sequence shared by all
 *     attention layers; pages return to the free list when a sequence is closed and are handed out again),
 *   - state slots for the recurrent layers (one slot per live sequence, reused the same way),
 *   - the step function, the continuous-batching generation loop on top of it and the on-device sampler.
 * Conventions as in ti_b200.h: 0 = success, ti_seq_last_error() has the message, no CPU fallback, opaque 64-bit handles.
 * Linear weights are [out, in] row-major and applied as W x.
 */
#ifndef TI_B200_SEQ_H
#define TI_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t ti_seq_model_t;

enum { TI_SEQ_MIXER_ATTENTION = 0, TI_SEQ_MIXER_WKV = 1 };
enum { TI_SEQ_ACT_RELU = 0, TI_SEQ_ACT_SILU = 1, TI_SEQ_ACT_GELU_TANH = 2 };
enum { TI_SEQ_BF16 = 0, TI_SEQ_F32 = 1 };   /* compute mode of a model, and element type of a tensor handed to set_tensor */

typedef struct ti_seq_layer_desc {
    int32_t mixer;           /* TI_SEQ_MIXER_* */
    int32_t heads, kv_heads; /* query heads, key/value heads (wkv: heads only) */
    int32_t dim, vdim;       /* per-head query/key size, value size (wkv: dim only) */
    int32_t window;          /* attention: a position sees itself and the window - 1 before it; 0 = everything before it */
    int32_t rot_dims;        /* leading coordinates of each head that are rotated, paired (2i, 2i+1); 0 = no rotation */
    float rot_base;
    int32_t rot_scaled;      /* 1: wavelength-dependent slow-down of the frequencies with the four numbers below */
    float rot_factor, rot_low, rot_high, rot_original;
    int32_t qk_norm;         /* 1: q and k are divided by their RMS per head after rotation */
    int32_t out_gate;        /* 1: head output times sigmoid of a per-head projection of the mixer input */
    float scale;             /* attention score scale */
    int32_t decay_rank;      /* wkv: inner size of the decay's two-matrix projection */
    int32_t ff;              /* feed-forward inner size, 0 = the layer has no feed-forward */
    int32_t ff_act;          /* TI_SEQ_ACT_* of the gate branch */
} ti_seq_layer_desc;

typedef struct ti_seq_model_desc {
    int32_t vocab, width, n_layers;
    int32_t loop_start, loop_stop, loop_times; /* layers [start, stop) run `times` times with the same weights and their own
                                                  cache / state per pass, each pass entered through the input projection of
                                                  [x; embedding]; times = 0: no looped block */
    float norm_eps, logit_scale;
    int32_t mode;            /* TI_SEQ_BF16 / TI_SEQ_F32 */
    int32_t max_tokens;      /* tokens the page pool holds (each sequence's count rounds up to whole pages) */
    int32_t max_seqs;        /* state slots = sequences that can be live at once */
} ti_seq_model_desc;

int ti_seq_init(int device);
const char* ti_seq_last_error(void);
uint64_t ti_seq_launch_count(void);

int ti_seq_model_new(const ti_seq_model_desc* desc, const ti_seq_layer_desc* layers, ti_seq_model_t* out);
/* tensor names: "embed", "loop.in", "final.norm", "head", "l<i>.norm1|norm1b|norm2|norm2b", "l<i>.mix.<x>", "l<i>.mlp.<x>";
 * `dtype` is the element type of `data` (TI_SEQ_BF16: raw bfloat16 bits, TI_SEQ_F32) */
int ti_seq_model_set_tensor(ti_seq_model_t m, const char* name, int32_t dtype, const void* data, const int64_t* shape, int32_t ndim);
/* uniform(-amp, amp) + offset generated on the device from (seed, element index): benchmark-size models */
int ti_seq_model_set_tensor_synthetic(ti_seq_model_t m, const char* name, const int64_t* shape, int32_t ndim, uint64_t seed, float amp,
                                      float offset);
/* number of tensors the description requires, and the name / shape of the i-th */
int ti_seq_model_tensor_count(ti_seq_model_t m, int32_t* n);
int ti_seq_model_tensor_info(ti_seq_model_t m, int32_t i, char* name, size_t cap, int64_t* shape, int32_t* ndim);
int ti_seq_model_finalize(ti_seq_model_t m);
int ti_seq_model_free(ti_seq_model_t m);

/* a sequence takes a state slot when opened; its pages are allocated as its tokens arrive; close gives both back */
int ti_seq_open(ti_seq_model_t m, int32_t* seq);
int ti_seq_close(ti_seq_model_t m, int32_t seq);
int ti_seq_length(ti_seq_model_t m, int32_t seq, int32_t* tokens);
int ti_seq_pool_info(ti_seq_model_t m, int32_t* free_pages, int32_t* total_pages, int32_t* free_slots, int32_t* page_tokens);
/* physical pages of a sequence (for tests of page reuse); returns the count in *n */
int ti_seq_pages(ti_seq_model_t m, int32_t seq, int32_t* pages, int32_t cap, int32_t* n);

/* One step: entry e brings counts[e] tokens of sequence seqs[e] (tokens are concatenated in `tokens`).  want_rows are row
 * indices into the concatenated tokens whose logits are copied to logits_host [n_want][vocab] (may be 0 / NULL). */
int ti_seq_step(ti_seq_model_t m, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens, int32_t n_want,
                const int32_t* want_rows, float* logits_host);
/* The same step, then a token is sampled on the device from the logits of each entry's LAST row (temperature 0 = greedy
 * arg-max; top_k 0 = no top-k; top_p 1 = no nucleus cut); sample_index[e] is the RNG counter of that pick. */
int ti_seq_step_sample(ti_seq_model_t m, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens,
                       float temperature, int32_t top_k, float top_p, uint64_t seed, const int32_t* sample_index, int32_t* out_tokens,
                       float* out_logprobs);

/* Continuous-batching generation: n_req prompts (concatenated in `prompts`, lens[i] tokens each), up to max_new new tokens
 * each.  Requests are admitted while a state slot and pages are free; every step runs the decode tokens of the running
 * requests plus prompt portions up to `step_tokens` rows in total; a request ends at max_new tokens or on eos (eos < 0: never).
 * out_tokens [n_req][max_new], out_lens [n_req]. */
int ti_seq_generate(ti_seq_model_t m, int32_t n_req, const int32_t* prompts, const int32_t* lens, int32_t max_new, int32_t step_tokens,
                    float temperature, int32_t top_k, float top_p, uint64_t seed, int32_t eos, int32_t* out_tokens, int32_t* out_lens);

/* debugging / tests: when enabled, every step keeps the residual stream after each layer run; read gives
 * [layer runs][rows of the last step][width] */
int ti_seq_debug_layers(ti_seq_model_t m, int32_t enable);
int ti_seq_debug_layers_read(ti_seq_model_t m, float* out, size_t cap_floats, int32_t* runs, int32_t* rows);
/* CUDA-event time of the last step (device work only), ms */
int ti_seq_last_step_ms(ti_seq_model_t m, float* ms);
/* writes a buffer larger than L2 (benchmarks: cold caches between timed steps) */
int ti_seq_flush_l2(void);
/* bytes of weights one step streams (every matrix once) and bytes of cache + state per cached token / per sequence */
int ti_seq_model_bytes(ti_seq_model_t m, double* weight_bytes, double* kv_bytes_per_token, double* state_bytes_per_seq);

#ifdef __cplusplus
}
#endif
#endif
