// Internal (C++) declarations shared by the .cu translation units.  The public C ABI is
// include/fasttalk_b200.h.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fasttalk_b200.h"

namespace ft {

constexpr int GEMM_MAX_SPLITS = 16;

// Per-device bookkeeping.  cudaFuncSetAttribute and the SM count belong to a DEVICE; a host may drive
// several GPUs from one process (the C ABI allows it), so "done once" flags are kept per device ordinal.
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0) d = 0;
    return d % kMaxDevices;
}
// Usage: `if (!flag.done()) { ...set the attributes...; flag.mark(); }` — the flag is raised only AFTER the
// set-up succeeded, so a second thread either sees it done or repeats the (idempotent) set-up itself.
struct PerDeviceFlag {
    volatile unsigned char flags[kMaxDevices] = {};
    bool done() const { return flags[current_device_slot()] != 0; }
    void mark() {
        __sync_synchronize();
        flags[current_device_slot()] = 1;
    }
};

// ---- gemm.cu
int make_tmap_bf16_k64(CUtensorMap* map, const void* base, int rows, int K, int box_rows);
int make_tmap_f16_3d(CUtensorMap* map, const void* base, int d0, int d1, int d2, int b0, int b1, int b2);
int gemm_pick_bn(int T, bool hilo);
bool gemm_pair_eligible(int n_out, int T);
bool gemm_f16_path_ok(int n_out, int T, int K, int splits);      // is there a one-fp16-plane form (x_planes = 3) of this launch?      // would launch_gemm run this (hi/lo, unsplit) projection on the CTA-pair kernel?
int gemm_pick_splits(int n_out, int T, int K, int num_sms, bool hilo);
size_t gemm_scratch_floats(int n_out, int T, int splits, bool hilo);   // split-K slabs of one launch
// Modes and fields: ft_gemm_epilogue in include/fasttalk_b200.h.
// mx_half / mx_lo_half: the same activations with 64-row boxes (only used with bn == 128, for the CTA-pair kernel)
int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap* mx_lo, int bn, int n_out,
                int T, int K, int splits, const ft_gemm_epilogue& epi, bool pdl, cudaStream_t stream,
                const CUtensorMap* mx_half = nullptr, const CUtensorMap* mx_lo_half = nullptr);

// ---- elementwise.cu
int launch_add_rmsnorm(float* resid, const float* partials, int n_splits, size_t split_stride,
                       const int* embed_tokens, const void* embed_table, const void* norm_w,
                       void* xn_out, void* xn_lo, const int* row_idx, int T, int h, float eps, bool pdl,
                       cudaStream_t stream);
int launch_rope_kv_append(const float* qkv, int n_splits, size_t split_stride, const float* cos_t,
                          const float* sin_t, const int* positions, const int* seq_slots,
                          const int* page_table, int max_pages, void* q_out, void* kv_layer, int T,
                          int nq, int nkv, int d, bool pdl, cudaStream_t stream);
int launch_embed_planes(const int* tokens, const void* embed, const void* gamma, float* resid, void* out,
                        void* out_lo, float* ssq, int ssq_parts, int ssq_stride, int T, int h, bool pdl,
                        cudaStream_t stream);
int launch_gather_planes(const void* x, const void* x_lo, const float* ssq, int ssq_parts, int ssq_stride,
                         const int* row_idx, int n_rows, int h, void* out, void* out_lo, float* ssq_out,
                         int ssq_out_stride, bool pdl, cudaStream_t stream);
int launch_planes_to_f16(const void* hi, const void* lo, void* out, size_t n_elems, bool pdl, cudaStream_t stream);
int launch_silu_mul(const float* gu, int n_splits, size_t split_stride, void* act, void* act_lo, int T,
                    int f, bool pdl, cudaStream_t stream);

// ---- attention.cu
size_t attn_decode_scratch_floats(int B, int nkv, int group, int d, int n_ctas);
int attn_decode_ctas_per_sm(int d);      // resident CTAs of the decode kernel per SM (<= 0: error)
const char* last_error();
int launch_attn_decode_plan(const int* ctx_lens, int* tile_prefix, int B, int nkv, float* scratch, bool pdl,
                            cudaStream_t stream);
int launch_attn_decode(const void* q, const void* kv_layer, const int* page_table, int max_pages,
                       const int* ctx_lens, const int* tile_prefix, void* out, void* out_lo, float* scratch,
                       int B, int nq, int nkv, int d, int n_ctas, bool pdl, cudaStream_t stream,
                       cudaEvent_t ev0 = nullptr, cudaEvent_t ev1 = nullptr, bool early = false);
// q_rows: rows (tokens) the q / out buffers hold — the tcgen05 kernel builds a tensor map over q; <= 0 = unknown,
// which selects the mma.sync kernel
int launch_attn_prefill(const void* q, const void* kv_layer, const int* page_table, int max_pages,
                        const int* req_q_start, const int* req_slot, const int* req_pos0,
                        const int* tile_req, const int* tile_q0, int n_tiles, void* out, void* out_lo, int nq,
                        int nkv, int d, bool pdl, cudaStream_t stream, int q_rows = 0);

// ---- attention_tc.cu (tcgen05 / TMEM prefill attention: head_dim 64 / 128, GQA group 3 / 4)
bool attn_prefill_tc_supported(int nq, int nkv, int d);
int launch_attn_prefill_tc(const void* q, int q_rows, const void* kv_layer, const int* page_table, int max_pages,
                           const int* req_q_start, const int* req_slot, const int* req_pos0, const int* tile_req,
                           const int* tile_q0, int n_tiles, void* out, void* out_lo, int nq, int nkv, int d, bool pdl,
                           cudaStream_t stream);

// ---- layered.cu (the layered model family: every size is a run-time value, activations fp32, weights bf16)
enum { LIN_PLAIN = 0, LIN_SWIGLU_PAIR = 1, LIN_SOFTCAP = 2, LIN_RELU2 = 3 };
// C[r, n] = sum_k A[row(r), k] * W[p][n, k] for problems p = 0..P-1.
//   batched (seg == null): every problem has rows 0..M-1; problem p reads A + p * a_col_stride, W + p * w_stride and
//                          writes C + p * c_col_stride (heads side by side in the columns of one buffer)
//   grouped (seg != null): problem p owns rows seg[p]..seg[p+1]-1 of C; row r reads A row a_rows[r] (or r)
// LIN_SWIGLU_PAIR: W rows (2j, 2j+1) are (gate_j, up_j); C[r, j] = silu(gate) * up, ldc counts those N/2 columns.
// LIN_SOFTCAP:     C = cap * tanh(C / cap).
// LIN_RELU2:       C = max(C, 0)^2.
struct LinearArgs {
    const float* A = nullptr;
    const int* a_rows = nullptr;
    const __nv_bfloat16* W = nullptr;
    float* C = nullptr;
    const int* seg = nullptr;
    long long w_stride = 0;
    int lda = 0, ldw = 0, ldc = 0, a_col_stride = 0, c_col_stride = 0;
    int M = 0, N = 0, K = 0, P = 1, epi = LIN_PLAIN;
    float cap = 0.f;
};
// rows_bound: M when batched; an upper bound of seg[P] when grouped
int launch_linear(const LinearArgs& a, int rows_bound, cudaStream_t stream);
// hi / lo (may be null): the normed row once more as bf16 planes, the input form of the tensor-core projections
// gain_w (may be null): a gain per coordinate instead of the single `gain`
int launch_embed_norm(const int* tokens, const void* embed, float* x, float* hn, void* hi, void* lo, int T, int W, float eps,
                      float gain, const float* gain_w, cudaStream_t stream);
int launch_to_planes(const float* x, void* hi, void* lo, size_t n, cudaStream_t stream);
int launch_softcap(float* x, size_t n, float cap, cudaStream_t stream);
int launch_gather_planes_rows(const float* src, const int* idx, void* hi, void* lo, int n, int W, cudaStream_t stream);
// act FT_ACT_SWIGLU: gu holds (gate, up) pairs, n counts pairs; FT_ACT_RELU2: gu holds n plain values
int launch_swiglu_planes(const float* gu, void* hi, void* lo, size_t n, cudaStream_t stream, int act = FT_ACT_SWIGLU);
int launch_combine_norm(float* x, float* hn, const float* proj, int ldp, int o_rg1, int o_rg2, const float* rg_bias,
                        const float* mix, const float* eout, const float* wt, const int* slot_pos, int top, int T, int W,
                        float eps, float gain, void* hi, void* lo, cudaStream_t stream);
int launch_gather_rows(const float* src, const int* idx, float* dst, int n, int W, cudaStream_t stream);
// cache16 (may be null): a bf16 copy of the latents, what the tensor-core attention reads
int launch_latent_write(const float* proj, int ldp, int o_dkv, const float* w, float* cache, void* cache16, const int* positions,
                        const int* seq_rows, const int* page_table, int max_pages, int rank, float eps, int T,
                        cudaStream_t stream);
// With fewer than kLatentSplitPairs (token, head) pairs in a step the keys of each are cut into up to kLatentMaxSplits
// shares that run side by side; `part` then holds pairs x shares x (kv_rank + 2) floats (null: never split).
constexpr int kLatentSplitPairs = 2048, kLatentMaxSplits = 8;
int latent_attn_splits(int T, int H);
// With cache16 and a latent size the tensor-core kernel is built for (latent_attn_mma_ok) the attention runs on mma.sync
// from bf16 operands; otherwise on the CUDA cores in fp32.
bool latent_attn_mma_ok(int rank);
int launch_latent_attn(const float* qlat, const float* cache, const void* cache16, const float* proj, int ldp, int o_gate,
                       float* out, float* part, const int* positions, const int* seq_rows, const int* page_table, int max_pages,
                       int H, int rank, float scale, int T, cudaStream_t stream);
struct DeltaArgs {
    const float* proj = nullptr;      // [T][ldp]: raw q | k | v at column o_q, beta logits at o_beta
    int ldp = 0, o_q = 0, o_beta = 0;
    const float* conv = nullptr;      // fp32 [channels][taps], last column = current token
    const float* araw = nullptr;      // [T][heads*dim] decay pre-activation (before dt_bias)
    const float* dt_bias = nullptr;   // [heads*dim]
    const float* a_log = nullptr;     // [heads]
    float* qkv = nullptr;             // out [T][channels]
    float* decay = nullptr;           // out [T][heads*dim] (may alias araw)
    float* beta = nullptr;            // out [T][heads]
    float* o = nullptr;               // out [T][heads*vdim]
    float* state = nullptr;           // slots of slot_stride floats; this layer's S at s_off, its tails at tail_off
    long long slot_stride = 0, s_off = 0, tail_off = 0;
    const int* seq_rows = nullptr;    // [T] request of a token
    const int* req_start = nullptr;   // [n_req + 1] first row of a request
    const int* req_pos0 = nullptr;    // [n_req] position of that row in its sequence
    const int* req_slot = nullptr;    // [n_req] state slot
    int heads = 0, kvh = 0, dim = 0, vdim = 0, taps = 0;
    int head_decay = 0;               // 1: araw holds one value per head (row stride ld_araw), dt_bias is [heads]
    int ld_araw = 0;
};
// prep (convolutions, norms, decays) -> tails -> recurrence -> output norm and gate (in place in a.o)
// gate rows have stride ldg (0: heads * vdim); gate_act 0: sigmoid, 1: silu
int launch_delta(const DeltaArgs& a, const float* gate, const float* out_norm, float eps, int T, int n_req,
                 cudaStream_t stream, int ldg = 0, int gate_act = 0);
int launch_route(const float* proj, int ldp, int o_router, int E, int top, int groups, int keep, int* ids, float* wts,
                 int* seg, int* slot_token, int* slot_pos, int T, cudaStream_t stream, int route_kind = FT_ROUTE_SOFTMAX,
                 int normalise = 0, float scale = 1.f);

// ---- branches.cu (branch mixers and the sandwich layer form: ft_branch_desc, FT_LAYER_SANDWICH; everything fp32)
// x += rms(y) * post_w;  hn = rms(x) * next_w  with  y = s0 * y0 + s1 * y1 + sum_k wt[t, k] * eout[slot_pos[t, k]]
// (each of the three parts optional); hi / lo (may be null): hn once more as bf16 planes.
struct SandwichArgs {
    float* x = nullptr;
    float* hn = nullptr;
    void *hi = nullptr, *lo = nullptr;
    const float *y0 = nullptr, *y1 = nullptr;
    float s0 = 1.f, s1 = 1.f;
    const float* eout = nullptr;
    const float* wt = nullptr;
    const int* slot_pos = nullptr;
    int top = 0;
    const float *post_w = nullptr, *next_w = nullptr;
    int W = 0;
    float eps = 0.f;
};
int launch_sandwich_norm(const SandwichArgs& a, int T, cudaStream_t stream);
int launch_silu_cols(float* x, int ld, int c0, int n, int T, cudaStream_t stream);
int launch_const_decay(const float* decay, float* ab, int heads, int T, cudaStream_t stream);
int launch_ff_act(const float* in, float* out, size_t n, int act, cudaStream_t stream);

// Softmax attention over the last `window` positions (0 = all) of a paged cache whose rows hold, per position,
// [G * dim rotated keys | G * vdim values].  launch_window_attention writes the step's rows first, then attends.
struct WindowArgs {
    const float* proj = nullptr;
    int ldp = 0, o_q = 0, o_k = 0, o_v = -1;      // o_v < 0: the values are the keys before rotation
    const float *q_bias = nullptr, *k_bias = nullptr, *rot_freq = nullptr;
    int rot_dims = 0;
    float* q_out = nullptr;                       // [T][H * dim] work buffer
    float* cache = nullptr;                       // this layer's [pages][64][G * (dim + vdim)]
    const int *positions = nullptr, *seq_rows = nullptr, *page_table = nullptr;
    int max_pages = 0;
    int H = 0, G = 0, dim = 0, vdim = 0, window = 0;
    float scale = 1.f, softcap = 0.f;
    float* out = nullptr;                         // [T][H * vdim]
    // options, off by default
    int qk_norm = 0;                              // q and k divided by their root mean square per head (before rotation)
    float eps = 0.f;
    int keep_first = 0;                           // positions below this stay visible beyond the window
    const float* sink = nullptr;                  // [H]: exp(sink) joins the softmax denominator
    const float* rel = nullptr;                   // [rel_n][H]: bias by distance, the last row for every larger distance
    int rel_n = 0;
    const float* v_bias = nullptr;                // [G * vdim]
    int v_role = 0;                               // 1: values also go to v_first; 2: v <- (1 - v_mix) v + v_mix v_first
    const float* v_mix = nullptr;                 // [1]
    float* v_first = nullptr;                     // [T][G * vdim] of the step
    int v_in_key = -1;                            // >= 0: the value of a key head is columns v_in_key .. + vdim of its (rotated) key;
                                                  // the cache row then holds the keys only
    // qk_norm 2: one root mean square over all query heads and one over all key heads.  q_gain / k_gain: gains on the normed
    // vectors, [dim] shared by the heads (qk_norm 1) or [H * dim] / [G * dim] (qk_norm 2)
    const float *q_gain = nullptr, *k_gain = nullptr;
    int rot_half = 0;                             // rotated pairs (i, i + rot_dims / 2) instead of (2i, 2i + 1)
    float rot_mag = 1.f;                          // factor on cos and sin
    int chunked = 0;                              // position p sees the keys from (p / window) * window on, not the last `window`
    int no_kv = 0;                                // the cache belongs to another layer, which has written the step's rows: queries only
};
// The step's prompt portions as the batch builder lists them: 64-token query tiles (request, first token), and per request
// its first row in the step, its page-table row and the position of its first token.
struct WindowTiles {
    const int *tile_req = nullptr, *tile_q0 = nullptr, *req_q_start = nullptr, *req_slot = nullptr, *req_pos0 = nullptr;
    int n_tiles = 0;
};
// n_single: how many of the step's first rows are single tokens of running sequences (they precede the portions)
int launch_window_attention(const WindowArgs& a, int T, int n_single, const WindowTiles& tm, cudaStream_t stream);

// S <- a_t S + b_t k_t v_t^T, o_t = S^T q_t per (request, head) over the request's rows in order; S [dim][vd] of head h at
// state + slot * slot_stride + s_off + h * dim * vd, zero at a sequence's start (req_pos0 == 0).
struct RecurArgs {
    const float *q = nullptr, *k = nullptr, *v = nullptr;      // rows of stride ldq / ldk / ldv; q, k: qk_heads x dim, v: heads x vd
    int ldq = 0, ldk = 0, ldv = 0;
    const float* ab = nullptr;                    // [T][heads][2]
    float* o = nullptr;                           // rows of stride ldo: heads x vd
    int ldo = 0;
    float* state = nullptr;
    long long slot_stride = 0, s_off = 0;
    const int *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
    int heads = 0, qk_heads = 0, dim = 0, vd = 0;
    int lanes = 0;                                // lanes per state column: 4, 8, 16, 32, or 0 = chosen by the launcher
};
// T: tokens of the step, a hint for the choice of lanes
int launch_decay_rule(const RecurArgs& a, int n_req, int T, cudaStream_t stream);

struct MemoryArgs {                               // gated matrix memory: what precedes the rule
    const float* proj = nullptr;
    int ldp = 0, o_v = 0, o_i = 0, o_f = 0;
    const float* gate_bias = nullptr;             // [2 * heads]
    float cap = 0.f;
    int heads = 0, vdim = 0;
    float* v_ext = nullptr;                       // out [T][heads][vdim + 1]
    float* gates = nullptr;                       // out [T][heads][2]: log input gate, log forget gate
    float* ab = nullptr;                          // out [T][heads][2]
    float* floor = nullptr;                       // out [T][heads]: exp(-m_t)
    float* state = nullptr;
    long long slot_stride = 0, m_off = 0;         // m [heads] of this layer inside a slot
    const int *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
};
int launch_memory_prep(const MemoryArgs& a, int T, int n_req, cudaStream_t stream);

struct SpaceArgs {                                // state space: convolution + SiLU, step sizes and decays, new tails
    const float* proj = nullptr;
    int ldp = 0, o_x = 0, o_dt = 0, channels = 0, taps = 0, heads = 0;
    const float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *a_log = nullptr;
    float* xbc = nullptr;                         // out [T][channels]
    int act = 1;                                  // 1: SiLU on the convolution's result; 0: the result as it is
    float* ab = nullptr;                          // out [T][heads][2] (heads == 0: no step sizes or decays are formed)
    float* state = nullptr;
    long long slot_stride = 0, tail_off = 0;      // tails [channels][taps - 1] of this layer inside a slot
    const int *seq_rows = nullptr, *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
};
int launch_space_prep(const SpaceArgs& a, int T, int n_req, cudaStream_t stream);

struct ReadoutArgs {
    const float* o = nullptr;                     // rows of stride ldo: heads x vd
    int ldo = 0, vd = 0, vdim = 0, heads = 0;
    float q_scale = 1.f;
    const float* floor = nullptr;                 // non-null: column vdim of every head is the normaliser
    const float* skip = nullptr;                  // [heads], with x rows of stride ldx
    const float* x = nullptr;
    int ldx = 0;
    const float* gate = nullptr;                  // rows of stride ldg
    int ldg = 0, gate_kind = 0;                   // 0 none, 1 silu before the norm, 2 sigmoid after it
    int norm_groups = 1;
    const float* gain = nullptr;                  // [heads * vdim]
    float eps = 0.f;
    float* out = nullptr;                         // [T][heads * vdim]
};
int launch_readout(const ReadoutArgs& a, int T, cudaStream_t stream);

// ---- postnorm.cu (FT_LAYER_POSTNORM: input convolutions, normed sublayer results, the weighted sum over depth; and the
// staging of latent window attention)
// x[t] = embed[token] * scale; the same row into hist (X_0) when given
int launch_embed_scale(const int* tokens, const void* embed, float scale, float* x, float* hist, int T, int W, cudaStream_t stream);
// What a sublayer reads: hn[t] = x[t] + sum_j w[:, j] x[t - taps + 1 + j] over the rows of t's own sequence; rows before the
// step come from the slot's ring [taps - 1][W] at tail_off, where the row of position p sits at p % (taps - 1) (zeros before
// position 0).  hi / lo (may be null): hn as planes.  w null: hn = x.  The ring is written by launch_postnorm.
struct CanonArgs {
    const float* x = nullptr;
    float* hn = nullptr;
    void *hi = nullptr, *lo = nullptr;
    const float* w = nullptr;                     // [W][taps]
    int taps = 0, W = 0;
    const float* state = nullptr;
    long long slot_stride = 0, tail_off = 0;
    const int *seq_rows = nullptr, *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
};
int launch_canon(const CanonArgs& a, int T, cudaStream_t stream);
// x_out = x + rms(y0 + b0 [+ y1 + b1]) * post_w (x_out may be x unless cw is given).
//   save_off >= 0: the last taps - 1 rows of x of every sequence (what the sublayer read) go into the ring at save_off first.
//   hist: the new row is X_k (written to hist[k]) and x_out becomes sum_{j <= k} depth_w[j] hist[j]; hist is [n][t_stride][W].
//   cw:   the next sublayer's input hn (+ planes) = x_out + conv(x_out) with weights cw [W][taps], rows before the step from
//         the ring at read_off.
struct PostNormArgs {
    const float* x = nullptr;
    float* x_out = nullptr;
    const float *y0 = nullptr, *y1 = nullptr, *b0 = nullptr, *b1 = nullptr;
    float s0 = 1.f, s1 = 1.f;
    const float* post_w = nullptr;
    float* hist = nullptr;
    const float* depth_w = nullptr;
    int k = 0;
    long long t_stride = 0;
    int W = 0;
    float eps = 0.f;
    int taps = 0;
    float* state = nullptr;
    long long slot_stride = 0, save_off = -1, read_off = 0;
    const int *seq_rows = nullptr, *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
    const float* cw = nullptr;
    float* hn = nullptr;
    void *hi = nullptr, *lo = nullptr;
};
int launch_postnorm(const PostNormArgs& a, int T, cudaStream_t stream);
// out[i] = rms(x[rows ? rows[i] : i]) * w (gain per coordinate) or * gain
int launch_rms_rows(const float* x, const int* rows, const float* w, float gain, float* out, int n, int W, float eps,
                    cudaStream_t stream);
// dst[t][dst_off + c] = rms(src[t][src_off .. + n)) * w[c]: a run of columns normed to a place (rows of stride lds / ldd)
int launch_rms_cols(const float* src, int lds, int src_off, const float* w, float* dst, int ldd, int dst_off, int n, float eps,
                    int T, cudaStream_t stream);
// Latent window attention: the staging row [heads x (rot query part | room for the folded plain query)] [rot key part |
// normed latent] of every token, from the query projection q [T][heads][dim | rot] and the layer's projection
// (rank latent columns, then rot columns, at o_k; latent gain w)
int launch_latent_stage(const float* q, int heads, int dim, int rot, const float* proj, int ldp, int o_k, int rank, const float* w,
                        float eps, float* stage, int lds, int T, cudaStream_t stream);

// ---- hyper.cu (FT_LAYER_HYPER: streams joined by small matrices, layer norms; selective scan; experts that read scaled rows)
// One kernel per sublayer joint, one CTA per row.  With `tokens`: X_s = embed[token] * scale for every stream (a step's
// first joint).  Otherwise y = s0 * f0(y0) + s1 * f1(y1) + sum_k wt[t, k] * eout[slot_pos[t, k]] (every part optional;
// f_i = y_i / rms(y_i) * g_i when g_i is given, wt null = ones) and X_t <- sum_s mix[s][t] X_s + out[t] * y.  Then what reads
// the streams next: u = sum_s in_next[s] X_s (null: the plain sum), hn = (u - mean) / sqrt(var + eps) * nw + nb (+ planes).
struct HyperArgs {
    float* X = nullptr;                           // [T][S][W]
    int S = 1, W = 0;
    float eps = 0.f;
    const int* tokens = nullptr;
    const void* embed = nullptr;                  // bf16 [vocab][W]
    float embed_scale = 1.f;
    const float *y0 = nullptr, *y1 = nullptr, *g0 = nullptr, *g1 = nullptr;
    float s0 = 1.f, s1 = 1.f;
    const float *eout = nullptr, *wt = nullptr;
    const int* slot_pos = nullptr;
    int top = 0;
    const float *mix = nullptr, *out = nullptr;   // [S][S] (from, to), [S]; null: identity, ones
    const float* in_next = nullptr;               // [S]
    const float *nw = nullptr, *nb = nullptr;     // gain and bias of the norm that follows
    float* hn = nullptr;
    void *hi = nullptr, *lo = nullptr;
    float* sum_out = nullptr;                     // [T][W] or null: the plain sum of the new streams
};
int launch_hyper_joint(const HyperArgs& a, int T, cudaStream_t stream);
// dst[slot_pos[i]] = wt[i] * src[i / top] for the T * top (token, choice) pairs: the rows the experts read when a score scales
// its expert's input.  dst fp32 [pairs][W] and / or bf16 planes hi, lo.
int launch_scaled_rows(const float* src, const float* wt, const int* slot_pos, int top, float* dst, void* hi, void* lo, int pairs,
                       int W, cudaStream_t stream);
// Selective scan: per (request, channel c) over the request's rows in order
//   dt = softplus(dt_raw[t][c] + dt_bias[c]);  S[n] <- exp(-exp(a_log[c][n]) dt) S[n] + dt x[t][c] B[t][n]
//   out[t][c] = (sum_n S[n] C[t][n] + skip[c] x[t][c]) * silu(z[t][c])
// S [channels][N] of a slot at s_off, zero at a sequence's start.
struct ScanArgs {
    const float* x = nullptr;                     // [T][ldx] convolved inputs
    const float* dt_raw = nullptr;                // [T][ldd]
    const float *B = nullptr, *C = nullptr;       // rows of stride ldbc, N numbers each
    const float* z = nullptr;                     // rows of stride ldz
    int ldx = 0, ldd = 0, ldbc = 0, ldz = 0;
    const float *dt_bias = nullptr, *a_log = nullptr, *skip = nullptr;
    float* out = nullptr;                         // [T][channels]
    float* state = nullptr;
    long long slot_stride = 0, s_off = 0;
    const int *req_start = nullptr, *req_pos0 = nullptr, *req_slot = nullptr;
    int channels = 0, N = 0;
    int rows = 0;                                 // T, all requests' tokens of the step
    float* ws = nullptr;                          // room for long requests cut into segments, or null (every request in
    int ws_rows = 0;                              // order then): ws_rows x channels x (N + 1) floats
};
int selective_scan_ws_rows(int rows);             // the ws_rows a step of this many rows needs
int launch_selective_scan(const ScanArgs& a, int n_req, cudaStream_t stream);

// ---- sampling.cu
int launch_sample(const float* logits, int B, int V, const float* temperature, const int* top_k,
                  const float* top_p, const unsigned long long* seeds, int* out_tokens, bool pdl,
                  cudaStream_t stream);

}  // namespace ft
