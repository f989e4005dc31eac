// The engine: KV page allocator, session table with prefix reuse, continuous-batching
// scheduler (decode rows + chunked-prefill rows in the same step) and the model forward that
// strings the kernels together.  Host logic only — every FLOP runs in the kernels of
// gemm.cu / elementwise.cu / attention.cu / sampling.cu.  There is no CPU fallback.
#include "common.cuh"
#include "ft_internal.h"
#include "../../include/fasttalk_b200.h"

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <new>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace ft {

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

struct Session {
    unsigned long long key = 0;
    std::vector<int> pages;      // KV pages in position order
    std::vector<int> tokens;     // tokens whose K/V sit in the cache (positions 0..size-1)
    int slot = -1;               // recurrent-state slot (models with stateful mixers), -1 = none
    bool busy = false;
    bool close_pending = false;  // session_close arrived while its request was inside a running step
    long long last_used = 0;
};

enum ReqState { REQ_WAITING = 0, REQ_PREFILL = 1, REQ_DECODE = 2, REQ_DONE = 3 };

struct Request {
    long long id = 0;
    Session* sess = nullptr;
    std::vector<int> prompt;     // full token list of this turn
    int prefill_pos = 0;         // next prompt index to run through the model
    float temperature = 0.f, top_p = 1.f;
    int top_k = 0, max_new = 0, n_generated = 0, ignore_eos = 0;
    unsigned long long seed = 0;
    int state = REQ_WAITING;
    int last_token = -1;         // sampled but not yet fed back
    int logits_row = -1;         // row of the logits buffer in the latest step
    bool in_flight = false;      // part of the step that is on the GPU right now (the engine lock is released
                                 // while the step runs, so submit / cancel / close do not wait for the GPU)
    bool cancel_pending = false; // cancelled while in flight: finished as "cancelled" when the step returns
};

struct OutTok { long long req; int token; int finish; };

// host-pinned + device mirror of everything a step's kernels index
struct StepMeta {
    int* h = nullptr;
    int* d = nullptr;
    size_t ints = 0;
    // offsets (in ints).  Fixed-size arrays come first; the page table and the per-token arrays
    // are packed behind them at per-step offsets so one H2D copy moves only what the step uses.
    size_t o_ctx, o_qstart, o_rslot, o_rpos0, o_treq, o_tq0, o_lrow, o_temp, o_topk, o_topp, o_seed,
        o_xstart, o_xpos0, o_xslot,               // every request of the step, decode rows first: first row | position of it | state slot
        o_pt;                                     // fixed
    size_t o_tokens, o_pos, o_rows, upload_ints;  // set by layout_step()
    size_t o_tprefix, o_sampled;                  // device-side work areas (never uploaded)
};

static inline size_t align4(size_t n) { return (n + 3) & ~size_t(3); }
static void layout_step(StepMeta& m, int n_req, int max_pages, int T) {
    m.o_tokens = m.o_pt + align4((size_t)n_req * max_pages);
    m.o_pos = m.o_tokens + align4(T);
    m.o_rows = m.o_pos + align4(T);
    m.upload_ints = m.o_rows + align4(T);
}

struct Layered;

struct Engine {
    ft_engine_config cfg;
    ft_weights w;
    Layered* lay = nullptr;      // non-null: a layered model (ft_engine_create_layered) instead of the Llama field set
    std::vector<int> free_slots; // recurrent-state slots not owned by a session
    int dev = 0, sms = 148;
    cudaStream_t stream = nullptr;
    std::mutex mu;               // scheduler state; NOT held while a step's kernels run
    std::mutex step_mu;          // one step (or debug / timer call that uses the stream's buffers) at a time

    int q_dim, kv_dim, qkv_dim, group, max_pages, t_max, r_max, logit_rows;
    int attn_ctas = 0;
    int decode_prefill_cap = 0;            // prompt tokens admitted per step while sequences are decoding (0 = no cap)
    int prefill_planes = 2;                // activation planes of the multi-wave prefill GEMMs (1 = hi only, 3 = one fp16 plane)
    // prefill_planes == 3: fp16 copies of the four projections' weights and fp16 staging planes of their inputs
    void *w16_qkv = nullptr, *w16_o = nullptr, *w16_gu = nullptr, *w16_d = nullptr;
    void *x16_xn = nullptr, *x16_attn = nullptr, *x16_act = nullptr;
    std::vector<CUtensorMap> m16_wqkv, m16_wo, m16_wgu, m16_wd;
    CUtensorMap m16_xn[2], m16_attn[2], m16_act[2];      // token boxes of 128 and 64 rows
    size_t kv_layer_bytes = 0;

    // device buffers
    uint8_t* kv = nullptr;
    float* resid = nullptr;
    float* ssq = nullptr;          // [ssq_parts][t_max] partial sums of squares of the residual rows
    float* ssq_last = nullptr;     // [ssq_parts][rows_last] gathered for the LM-head rows
    int ssq_parts = 0, rows_last = 0;
    float* gemm_scratch = nullptr; // split-K slabs of the fused-epilogue GEMMs (one wave of CTAs)
    int* gemm_sync = nullptr;      // their arrival counters
    int sync_parity = 0;           // which word of each counter pair the next split-K launch uses
    // bf16 activations feeding the GEMMs are kept as hi + lo planes (see gemm.cu)
    void *xn = nullptr, *q = nullptr, *attn_out = nullptr, *act = nullptr, *xn_last = nullptr;
    void *xn_lo = nullptr, *attn_out_lo = nullptr, *act_lo = nullptr, *xn_last_lo = nullptr;
    float* logits = nullptr;
    float* attn_scratch = nullptr;
    StepMeta meta;

    // tensor parallelism (2 ranks): buffers the peer writes into, and the peer's as mapped here
    int tp = 1, vocab_local = 0;
    float* tp_xchg = nullptr;          // [2 parities][t_max][hidden] fp32 partial rows from the peer
    unsigned* tp_flags = nullptr;      // [kTpFlags] arrival words written by the peer
    float* peer_xchg = nullptr;
    unsigned* peer_flags = nullptr;
    float* peer_logits = nullptr;
    unsigned tp_epoch = 0;             // advances once per exchanging launch, identically on both ranks

    // tensor maps: weights per layer, activations per BN
    std::vector<CUtensorMap> m_wqkv, m_wo, m_wgu, m_wd;
    CUtensorMap m_lm;
    CUtensorMap m_xn[4], m_attn[4], m_act[4], m_last[4];              // token tiles 16/32/64/128
    CUtensorMap m_xn_lo[4], m_attn_lo[4], m_act_lo[4], m_last_lo[4];

    // scheduler state
    std::vector<int> free_pages;
    std::unordered_map<unsigned long long, Session*> sessions;
    std::unordered_map<long long, Request*> requests;
    std::deque<Request*> waiting;
    std::vector<Request*> active;
    std::deque<OutTok> out;
    long long next_req = 0, clock = 0;
    ft_engine_stats st = {};
    bool pdl = false;
    // optional CUDA-event timing of the decode-attention kernel (bench roofline)
    bool profile = false;
    std::vector<cudaEvent_t> prof_ev;      // 2 per layer
    int prof_used = 0;
    long long prof_ctx_sum = 0;            // sum of context lengths of the step's decode rows
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    // device time of every step (events on the engine stream around upload .. sampled-token copy)
    cudaEvent_t s0 = nullptr, s1 = nullptr;
    struct StepRec { float gpu_ms, n_decode, n_prefill, host_ms; };
    std::deque<StepRec> step_log;          // most recent kStepTimes steps, oldest first

    // the engine's own stepping thread (ft_engine_start): steps whenever something is runnable, so that no host
    // language sits between two steps; the owner only submits, waits for events and drains them
    std::thread loop_thread;
    bool loop_on = false, loop_stop = false;
    int loop_error = 0;
    std::string loop_error_msg;
    std::condition_variable cv_work;       // submit / cancel / stop -> the loop
    std::condition_variable cv_out;        // events queued, loop failed or stopped -> ft_engine_wait
    int waiters = 0;                       // threads inside ft_engine_wait
    bool closing = false;                  // ft_engine_destroy has begun: waiters leave, nobody new comes in
};

// A layered model inside the engine: the descriptors, the paged latent cache of its attention layers, the state slots
// of its recurrent layers and the fp32 work buffers of a step.
struct LayeredLayer {
    ft_layer_desc d;
    size_t cache_off = 0;              // floats: this layer's [num_pages][64][kv_rank] block in lat_cache
    size_t s_off = 0, tail_off = 0;    // floats inside a state slot: S [heads][dim][vdim], tails [channels][conv - 1]
    // branch mixers: per branch its block in kv_cache (window attention), its S inside a state slot, and what else it keeps
    // there (the running maximum of a matrix memory, the convolution tails of a state space)
    size_t br_cache_off[2] = {0, 0}, br_s_off[2] = {0, 0}, br_x_off[2] = {0, 0};
    size_t canon_off[2] = {0, 0};      // post-norm layers: the tails [taps - 1][width] of the two input convolutions in a slot
    int lender_branch[2] = {0, 0};     // window attention over another layer's cache: which branch of that layer owns it
};
struct Layered {
    ft_layered_model m;
    std::vector<LayeredLayer> layers;
    float* lat_cache = nullptr;
    void* lat_cache16 = nullptr;       // serving form: bf16 copy of the latents, same places (tensor-core attention)
    float* kv_cache = nullptr;         // window-attention branches: per layer [num_pages][64][kv_heads * (dim + vdim)] fp32
    float* state = nullptr;
    size_t slot_stride = 0;            // floats per state slot
    int n_stateful = 0;                // layers whose mixer carries state from token to token
    int ld_proj = 0, top_max = 0, scan_ws_rows = 0;
    float *hn = nullptr, *proj = nullptr, *b1 = nullptr, *b2 = nullptr, *b3 = nullptr, *b4 = nullptr, *beta = nullptr, *scan_ws = nullptr,
          *attn_part = nullptr, *mix = nullptr, *act = nullptr, *eout = nullptr, *wts = nullptr, *xlast = nullptr;
    // branch mixers and sandwich layers: queries, prepared values, rule outputs, read-out, (decay, input) pairs, log gates,
    // denominator floors, the second branch's projection, feed-forward halves, router logits
    float *bq = nullptr, *bv = nullptr, *bo = nullptr, *bfin = nullptr, *ab = nullptr, *gates = nullptr, *floor = nullptr,
          *mix2 = nullptr, *ffa = nullptr, *ffb = nullptr, *rlog = nullptr;
    int *ids = nullptr, *seg = nullptr, *slot_token = nullptr, *slot_pos = nullptr;
    void *pl_hi = nullptr, *pl_lo = nullptr;      // bf16 planes of a projection's input [t_max][k_max]
    void *hn_hi = nullptr, *hn_lo = nullptr;      // bf16 planes of the normed layer input [t_max][width]
    // experts on the tensor cores: planes of the gathered rows, fp32 gate/up results, planes of the activations, and the
    // segment table on the host (the per-expert launches need the row counts)
    void *mx_hi = nullptr, *mx_lo = nullptr, *ax_hi = nullptr, *ax_lo = nullptr;
    float* gu = nullptr;
    int* h_seg = nullptr;
    // the per-expert GEMMs are small (a few dozen CTAs): they are dealt over the engine's stream and three side streams
    static constexpr int kSide = 3;
    cudaStream_t side[kSide] = {};
    cudaEvent_t side_done[kSide] = {}, main_ready = nullptr;
    bool tensor = false;               // projections that tile run on the tensor cores (ft_layered_model.exact_f32 == 0)
    // post-norm layers: the stream as every layer left it [n_layers + 1][t_max][width] (the sum over depth reads them all), the
    // values of the first value-mixing attention layer of the step, the staging rows of latent window attention
    // resid2: the stream between a layer's two sublayers (the joint kernel that forms the feed-forward's input reads
    // neighbouring rows of the old stream while it writes the new one)
    float *hist = nullptr, *v_first = nullptr, *lstage = nullptr, *resid2 = nullptr;
    bool postnorm = false;
    // hyper-connected layers: the streams of a step [t_max][streams][width]
    float* streams = nullptr;
    bool hyper = false;
    float* trail = nullptr;            // debug: residual stream after every layer [n_layers][t_max][width]
    bool trail_on = false;
};
constexpr size_t kStepTimes = 4096;
constexpr int kDefaultPrefillPlanes = 3;      // one fp16 plane x fp16 weight copies in the large prefill GEMMs (measured: DESIGN.md §2)
constexpr int kGemmTokenTile = 128;             // token tile of the multi-tile projections (gemm_pick_bn)
constexpr int kDefaultDecodePrefillCap = 896;    // <= 128 decode rows + 896 -> 1024 rows: a 1B step of ~4.3 ms (1280 rows: 6.6 ms)

// Every entry point that touches CUDA makes the engine's device current for its duration: the caller may be a
// thread whose current device is another GPU (a fresh thread starts on device 0).
// Does `dev` have a live primary context in this process?  (driver API through the runtime's entry-point lookup; on
// any doubt: yes)
static bool primary_ctx_active(int dev) {
    typedef CUresult (*Fn)(CUdevice, unsigned int*, int*);
    static Fn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuDevicePrimaryCtxGetState", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<Fn>(p);
    }();
    unsigned int flags = 0;
    int active = 1;
    if (!fn || fn((CUdevice)dev, &flags, &active) != CUDA_SUCCESS) return true;
    return active != 0;
}

struct DeviceGuard {
    int prev = -1, dev;
    explicit DeviceGuard(int d) : dev(d) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        // Back to the caller's device — unless that is only the default of a thread that never touched a GPU: since
        // CUDA 12 cudaSetDevice creates the device's context, and "restoring" device 0 from a process that lives on
        // another GPU would build one there (0.4 s and ~0.5 GB on a GPU that belongs to another rank).
        if (prev >= 0 && prev != dev && primary_ctx_active(prev)) cudaSetDevice(prev);
    }
};
// The split-K rendezvous and the tensor-parallel flag wait spin inside kernels and need every CTA of a launch
// resident at once.  One engine alone on a GPU guarantees that (grids are sized to one wave); two engines in one
// process on the SAME GPU (two models behind one server) could each hold part of the SMs and wait for CTAs that
// can never be scheduled.  Steps are synchronous (they end with a stream synchronise), so serialising the steps
// of engines that share a device removes the hazard without costing a lone engine anything.
static std::mutex g_device_step_mu[kMaxDevices];

constexpr int kTpFlags = 16384;        // >= CTAs of any exchanging GEMM launch; the last word is the step barrier

// Step barrier between the two ranks before sampling: both halves of the logits are in place.
__global__ void tp_barrier_kernel(unsigned* peer_flag, const unsigned* flag, unsigned epoch) {
    if (threadIdx.x == 0) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(epoch) : "memory");
        unsigned v, spins = 0;
        do {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if ((int)(v - epoch) >= 0) break;
            __nanosleep(64);
            if (++spins > (1u << 25)) __trap();
        } while (true);
    }
}

static int bn_index(int bn) { return bn == 16 ? 0 : bn == 32 ? 1 : bn == 64 ? 2 : 3; }
static const int kBns[4] = {16, 32, 64, 128};

// ------------------------------------------------------------------ pages / sessions
static void release_pages_beyond(Engine* e, Session* s, int keep_tokens) {
    const int keep = ceil_div(keep_tokens, kKvTile);
    while ((int)s->pages.size() > keep) {
        e->free_pages.push_back(s->pages.back());
        s->pages.pop_back();
    }
    if ((int)s->tokens.size() > keep_tokens) s->tokens.resize(keep_tokens);
}

static void drop_session(Engine* e, Session* s) {
    release_pages_beyond(e, s, 0);
    if (s->slot >= 0) e->free_slots.push_back(s->slot);
    e->sessions.erase(s->key);
    delete s;
}

// Free pages by evicting idle sessions, least recently used first.
static bool reclaim_pages(Engine* e, int need) {
    while ((int)e->free_pages.size() < need) {
        Session* victim = nullptr;
        for (auto& kv : e->sessions)
            if (!kv.second->busy && !kv.second->pages.empty() &&
                (!victim || kv.second->last_used < victim->last_used))
                victim = kv.second;
        if (!victim) return false;
        release_pages_beyond(e, victim, 0);
    }
    return true;
}

static bool ensure_pages(Engine* e, Session* s, int n_tokens) {
    const int need = ceil_div(n_tokens, kKvTile) - (int)s->pages.size();
    if (need <= 0) return true;
    if ((int)e->free_pages.size() < need && !reclaim_pages(e, need)) return false;
    for (int i = 0; i < need; ++i) {
        s->pages.push_back(e->free_pages.back());
        e->free_pages.pop_back();
    }
    return true;
}

static void finish_request(Engine* e, Request* r, int reason, int token) {
    e->out.push_back({r->id, token, reason});
    r->state = REQ_DONE;
    if (r->sess) {
        r->sess->busy = false;
        r->sess->last_used = ++e->clock;
    }
}

// ------------------------------------------------------------------ forward
struct Batch {
    int n_decode = 0;                 // rows [0, n_decode): one token per sequence
    int T = 0;                        // total token rows
    int n_req = 0;                    // page-table rows (decode first, then prefill requests)
    int n_prefill_req = 0;
    int n_tiles = 0;                  // prefill attention q tiles
    int n_logit_rows = 0;
    bool logit_rows_identity = false; // logits wanted for rows 0..n_logit_rows-1 exactly (no gather)
};

#define FT_TRY(x)                                   \
    do {                                            \
        int _r = (x);                               \
        if (_r) return _r;                          \
    } while (0)

// One projection with a fused epilogue.  `staged` epilogues (RESID / QKV_ROPE) split K across
// one wave of CTAs that rendezvous in the epilogue; the others run unsplit.
struct F16Path {                 // the fp16 single-plane form of one projection (prefill_planes == 3); null maps = not available
    const CUtensorMap* mw = nullptr;
    const CUtensorMap* mx = nullptr;         // [2]: 128- and 64-row boxes
    const void *hi = nullptr, *lo = nullptr;
    void* x16 = nullptr;
    bool ready = false;                      // the producer's epilogue already wrote x16: no staging kernel
};

static int run_gemm(Engine* e, const CUtensorMap& mw, const CUtensorMap* xmaps, const CUtensorMap* xmaps_lo,
                    int T, int n_out, int K, ft_gemm_epilogue epi, const F16Path* f16 = nullptr) {
    const int bn = gemm_pick_bn(T, true);
    const bool staged = epi.mode == FT_EPI_RESID || epi.mode == FT_EPI_QKV_ROPE;
    const int splits = staged ? gemm_pick_splits(n_out, T, K, e->sms, true) : 1;
    epi.scratch = e->gemm_scratch;
    epi.sync = e->gemm_sync;
    epi.x_planes = e->prefill_planes == 3 ? 2 : e->prefill_planes;
    if (staged && splits > 1) {              // launches are stream-ordered and each epilogue waits for its predecessor
        epi.sync_mode = 1 + e->sync_parity;
        epi.sync_slots = e->sms;
        e->sync_parity ^= 1;
    }
    if (e->tp > 1 && epi.mode == FT_EPI_RESID) {
        // row-parallel projection: the all-reduce over the two ranks happens inside the epilogue
        const unsigned epoch = ++e->tp_epoch;
        const size_t half = (size_t)e->t_max * e->cfg.hidden;
        epi.tp_peer_xchg = e->peer_xchg + (epoch & 1) * half;
        epi.tp_xchg = e->tp_xchg + (epoch & 1) * half;
        epi.tp_peer_flags = e->peer_flags;
        epi.tp_flags = e->tp_flags;
        epi.tp_epoch = epoch;
        const int ctas = (n_out / 128) * ((T + bn - 1) / bn) * splits;
        FT_REQUIRE(ctas < kTpFlags, "engine: %d CTAs exceed the tensor-parallel arrival words", ctas);
    }
    e->st.kernel_launches++;
    if (f16 && f16->mw && e->prefill_planes == 3 && gemm_f16_path_ok(n_out, T, K, splits)) {
        // large prefill projection: ONE fp16 plane (= fp16(hi + lo), staged by a small kernel) against fp16 weights
        if (!f16->ready) {
            FT_TRY(launch_planes_to_f16(f16->hi, f16->lo, f16->x16, (size_t)T * K, e->pdl, e->stream));
            e->st.kernel_launches++;
        }
        epi.x_planes = 3;
        return launch_gemm(*f16->mw, f16->mx[0], &f16->mx[0], bn, n_out, T, K, 1, epi, e->pdl, e->stream, &f16->mx[1],
                           &f16->mx[1]);
    }
    return launch_gemm(mw, xmaps[bn_index(bn)], &xmaps_lo[bn_index(bn)], bn, n_out, T, K, splits, epi, e->pdl,
                       e->stream, &xmaps[bn_index(64)], &xmaps_lo[bn_index(64)]);
}

// The norm-deferred layer chain (5 kernels per layer):
//   QKV GEMM [x 1/rms, RoPE, KV append] -> attention -> O GEMM [resid +=, planes = resid*gamma_mlp, ssq]
//   -> gate/up GEMM [x 1/rms, SwiGLU] -> down GEMM [resid +=, planes = resid*gamma_next, ssq]
// `xn` planes always hold resid * gamma of the NEXT norm; `ssq` its per-row-tile sums of squares.
static int forward_layered(Engine* e, const Batch& b);

static int forward(Engine* e, const Batch& b) {
    if (e->lay) return forward_layered(e, b);
    const ft_engine_config& c = e->cfg;
    StepMeta& m = e->meta;
    int* d = m.d;
    const int T = b.T;
    const size_t H = c.hidden;
    auto bf16_off = [](const void* p, size_t elems) {
        return (const void*)((const uint8_t*)p + elems * 2);
    };
    FT_TRY(launch_embed_planes(d + m.o_tokens, e->w.embed, e->w.attn_norm, e->resid, e->xn, e->xn_lo, e->ssq,
                               e->ssq_parts, e->t_max, T, c.hidden, e->pdl, e->stream));
    e->st.kernel_launches++;
    if (b.n_decode > 0) {
        FT_TRY(launch_attn_decode_plan(d + m.o_ctx, d + m.o_tprefix, b.n_decode, c.n_kv_heads, e->attn_scratch,
                                       e->pdl, e->stream));
        e->st.kernel_launches++;
    }
    // L2 prefetch of the next projection's weights only pays when the GEMMs are latency-bound
    const bool decode_only = b.n_tiles == 0 && T <= 128;
    const bool use16 = e->prefill_planes == 3 && e->w16_qkv != nullptr && T > 128;
    // which projections take the one-fp16-plane form this step: their producers write that plane in their epilogues
    // (O -> gate/up input, down -> next QKV input, gate/up -> down input); layer 0's QKV input (embedding kernel) and the
    // attention output are staged by planes_to_f16 instead
    static const bool direct = getenv("FT_F16_STAGE_ALL") == nullptr;          // A/B switch: stage every plane with planes_to_f16
    const bool f16_qkv = direct && use16 && gemm_f16_path_ok(e->qkv_dim, T, c.hidden, gemm_pick_splits(e->qkv_dim, T, c.hidden, e->sms, true));
    const bool f16_gu = direct && use16 && gemm_f16_path_ok(2 * c.ffn, T, c.hidden, 1);
    const bool f16_d = direct && use16 && gemm_f16_path_ok(c.hidden, T, c.ffn, gemm_pick_splits(c.hidden, T, c.ffn, e->sms, true));
    ft_gemm_epilogue rstd = {};            // fields shared by every epilogue that applies 1/rms
    rstd.ssq_in = e->ssq;
    rstd.ssq_parts = e->ssq_parts;
    rstd.ssq_stride = e->t_max;
    rstd.inv_h = 1.f / (float)c.hidden;
    rstd.eps = c.rms_eps;
    for (int l = 0; l < c.layers; ++l) {
        uint8_t* kv_l = e->kv + (size_t)l * e->kv_layer_bytes;
        {
            ft_gemm_epilogue ep = rstd;
            ep.mode = FT_EPI_QKV_ROPE;
            ep.rope_cos = e->w.rope_cos;
            ep.rope_sin = e->w.rope_sin;
            ep.positions = d + m.o_pos;
            ep.seq_rows = d + m.o_rows;
            ep.page_table = d + m.o_pt;
            ep.max_pages = e->max_pages;
            ep.q_out = e->q;
            ep.kv_layer = kv_l;
            ep.nq = c.n_q_heads;
            ep.nkv = c.n_kv_heads;
            ep.head_dim = c.head_dim;
            const F16Path f = {use16 ? &e->m16_wqkv[l] : nullptr, e->m16_xn, e->xn, e->xn_lo, e->x16_xn, l > 0 && f16_qkv};
            FT_TRY(run_gemm(e, e->m_wqkv[l], e->m_xn, e->m_xn_lo, T, e->qkv_dim, c.hidden, ep, &f));
        }
        if (b.n_decode > 0) {
            cudaEvent_t ev0 = nullptr, ev1 = nullptr;
            if (e->profile) {
                ev0 = e->prof_ev[2 * l];
                ev1 = e->prof_ev[2 * l + 1];
                e->prof_used = l + 1;
            }
            FT_TRY(launch_attn_decode(e->q, kv_l, d + m.o_pt, e->max_pages, d + m.o_ctx, d + m.o_tprefix,
                                      e->attn_out, e->attn_out_lo, e->attn_scratch, b.n_decode, c.n_q_heads,
                                      c.n_kv_heads, c.head_dim, e->attn_ctas, e->pdl, e->stream, ev0, ev1,
                                      /*early=*/l > 0 && b.n_tiles == 0));
            e->st.kernel_launches++;
        }
        if (b.n_tiles > 0) {
            FT_TRY(launch_attn_prefill(e->q, kv_l, d + m.o_pt, e->max_pages, d + m.o_qstart, d + m.o_rslot,
                                       d + m.o_rpos0, d + m.o_treq, d + m.o_tq0, b.n_tiles, e->attn_out,
                                       e->attn_out_lo, c.n_q_heads, c.n_kv_heads, c.head_dim, e->pdl,
                                       e->stream, e->t_max));
            e->st.kernel_launches++;
        }
        {
            ft_gemm_epilogue ep = {};
            ep.mode = FT_EPI_RESID;
            ep.resid = e->resid;
            ep.gamma = bf16_off(e->w.mlp_norm, (size_t)l * H);
            ep.out = e->xn;
            ep.out_lo = e->xn_lo;
            ep.ssq_out = e->ssq;
            ep.ssq_stride = e->t_max;
            if (f16_gu) {           // the gate/up projection reads the fp16 plane alone: no hi / lo planes to write
                ep.out_f16 = e->x16_xn;
                ep.out = ep.out_lo = nullptr;
            }
            if (decode_only) {      // stream the gate/up weights into L2 behind this latency-bound kernel
                ep.prefetch = bf16_off(e->w.wgu, (size_t)l * 2 * c.ffn * H);
                ep.prefetch_bytes = (long long)2 * c.ffn * H * 2;
            }
            const F16Path f = {use16 ? &e->m16_wo[l] : nullptr, e->m16_attn, e->attn_out, e->attn_out_lo, e->x16_attn};
            FT_TRY(run_gemm(e, e->m_wo[l], e->m_attn, e->m_attn_lo, T, c.hidden, e->q_dim, ep, &f));
        }
        {   // gate/up projection: 1/rms and SwiGLU in the epilogue, act = silu(g) * u
            ft_gemm_epilogue ep = rstd;
            ep.mode = FT_EPI_SWIGLU;
            ep.out = e->act;
            ep.out_lo = e->act_lo;
            if (f16_d) {
                ep.out_f16 = e->x16_act;
                ep.out = ep.out_lo = nullptr;
            }
            if (decode_only) {
                ep.prefetch = bf16_off(e->w.wd, (size_t)l * c.ffn * H);
                ep.prefetch_bytes = (long long)c.ffn * H * 2;
            }
            const F16Path f = {use16 ? &e->m16_wgu[l] : nullptr, e->m16_xn, e->xn, e->xn_lo, e->x16_xn, f16_gu};
            FT_TRY(run_gemm(e, e->m_wgu[l], e->m_xn, e->m_xn_lo, T, 2 * c.ffn, c.hidden, ep, &f));
        }
        {
            ft_gemm_epilogue ep = {};
            ep.mode = FT_EPI_RESID;
            ep.resid = e->resid;
            ep.gamma = l + 1 < c.layers ? bf16_off(e->w.attn_norm, (size_t)(l + 1) * H) : e->w.final_norm;
            ep.out = e->xn;
            ep.out_lo = e->xn_lo;
            ep.ssq_out = e->ssq;
            ep.ssq_stride = e->t_max;
            if (f16_qkv && l + 1 < c.layers) {     // (the last layer's planes feed the LM head's row gather)
                ep.out_f16 = e->x16_xn;
                ep.out = ep.out_lo = nullptr;
            }
            if (decode_only && l + 1 < c.layers) {
                ep.prefetch = bf16_off(e->w.wqkv, (size_t)(l + 1) * e->qkv_dim * H);
                ep.prefetch_bytes = (long long)e->qkv_dim * H * 2;
            }
            const F16Path f = {use16 ? &e->m16_wd[l] : nullptr, e->m16_act, e->act, e->act_lo, e->x16_act, f16_d};
            FT_TRY(run_gemm(e, e->m_wd[l], e->m_act, e->m_act_lo, T, c.hidden, c.ffn, ep, &f));
        }
    }
    if (b.n_logit_rows > 0) {
        // LM head on the rows that need logits (all of them in a pure decode step)
        const CUtensorMap* xm = e->m_xn;
        const CUtensorMap* xl = e->m_xn_lo;
        ft_gemm_epilogue ep = rstd;
        ep.mode = FT_EPI_LOGITS;
        ep.out = e->logits;
        if (!b.logit_rows_identity) {
            FT_TRY(launch_gather_planes(e->xn, e->xn_lo, e->ssq, e->ssq_parts, e->t_max, d + m.o_lrow,
                                        b.n_logit_rows, c.hidden, e->xn_last, e->xn_last_lo, e->ssq_last,
                                        e->rows_last, e->pdl, e->stream));
            e->st.kernel_launches++;
            xm = e->m_last;
            xl = e->m_last_lo;
            ep.ssq_in = e->ssq_last;
            ep.ssq_stride = e->rows_last;
        }
        if (e->tp > 1) {                 // vocabulary-parallel: each rank fills its columns on both GPUs
            ep.out_stride = c.vocab;
            ep.out_col0 = c.tp_rank * e->vocab_local;
            ep.tp_peer_out = e->peer_logits;
        }
        FT_TRY(run_gemm(e, e->m_lm, xm, xl, b.n_logit_rows, e->vocab_local, c.hidden, ep));
        if (e->tp > 1) {
            const unsigned epoch = ++e->tp_epoch;
            tp_barrier_kernel<<<1, 32, 0, e->stream>>>(e->peer_flags + kTpFlags - 1, e->tp_flags + kTpFlags - 1, epoch);
            FT_CHECK_CUDA(cudaGetLastError());
            e->st.kernel_launches++;
        }
    }
    return 0;
}

// A plain projection C[T][N] = A[T][K] W[N][K]^T.  With enough rows and shapes that tile, on the tensor cores: the fp32 input
// as bf16 hi + lo planes (`hi` / `lo` if the producer already wrote them, else staged here), fp32 out.  Otherwise, and always
// in the exact-fp32 form, the CUDA-core kernels.
constexpr int kTensorMinRows = 9;
constexpr int kFuseCanonRows = 256;          // steps up to this many rows form the feed-forward's input inside the post-norm kernel
constexpr int kMoeTensorMinPairs = 256;      // (token, choice) pairs from which the experts run as per-expert tensor-core GEMMs
static int dense(Engine* e, const float* A, const void* hi, const void* lo, const void* W, float* C, int T, int N, int K,
                 float softcap = 0.f) {
    Layered& L = *e->lay;
    if (L.tensor && T >= kTensorMinRows && N % 128 == 0 && K % 64 == 0) {
        if (!hi) {
            FT_TRY(launch_to_planes(A, L.pl_hi, L.pl_lo, (size_t)T * K, e->stream));
            e->st.kernel_launches++;
            hi = L.pl_hi;
            lo = L.pl_lo;
        }
        ft_gemm_epilogue ep = {};
        ep.mode = FT_EPI_PARTIAL;
        ep.out = C;
        FT_TRY(ft_gemm_fused(W, hi, lo, N, T, K, 1, &ep, e->stream));
        e->st.kernel_launches++;
        if (softcap > 0.f) {
            FT_TRY(launch_softcap(C, (size_t)T * N, softcap, e->stream));
            e->st.kernel_launches++;
        }
        return 0;
    }
    LinearArgs a;
    a.A = A; a.lda = K; a.W = (const __nv_bfloat16*)W; a.ldw = K; a.C = C; a.ldc = N; a.M = T; a.N = N; a.K = K;
    if (softcap > 0.f) { a.epi = LIN_SOFTCAP; a.cap = softcap; }
    FT_TRY(launch_linear(a, T, e->stream));
    e->st.kernel_launches++;
    return 0;
}

// The mixture of experts of one layer: routing from `logits` (row stride ldl, first column o_router), then every (token,
// choice) pair through its expert, grouped by expert.  Reads the rows of L.hn; leaves the pairs' outputs in L.eout and their
// weights / places in L.wts / L.slot_pos (the caller's residual kernel gathers them).
static int run_experts(Engine* e, const ft_layer_desc& c, const float* logits, int ldl, int o_router, int T) {
    Layered& L = *e->lay;
    const int W = L.m.width;
    cudaStream_t st = e->stream;
    auto launched = [&](int n = 1) { e->st.kernel_launches += n; };
    const bool sandwich = c.form == FT_LAYER_SANDWICH || c.form == FT_LAYER_HYPER;      // forms whose router is a matrix of its own
    const int act = sandwich ? c.ff_act : FT_ACT_SWIGLU;
    const int n_up = act == FT_ACT_SWIGLU ? 2 * c.ff : c.ff;          // rows of an expert's first matrix
    const bool scaled_in = c.route_input != 0;                        // the experts read score * row, in sorted order
    const int top = c.top;
    FT_TRY(launch_route(logits, ldl, o_router, c.experts, c.top, sandwich ? 1 : c.groups, sandwich ? 1 : c.keep, L.ids, L.wts,
                        L.seg, L.slot_token, L.slot_pos, T, st, sandwich ? c.route_kind : FT_ROUTE_SOFTMAX,
                        sandwich ? c.route_norm : 0, sandwich ? c.route_scale : 1.f));
    const int pairs = T * top;
    const bool on_tensor = L.tensor && pairs >= kMoeTensorMinPairs && n_up % 128 == 0 && c.ff % 64 == 0 && W % 128 == 0 &&
                           W % 64 == 0;
    if (on_tensor) {
        // One tcgen05 GEMM per expert over its run of sorted rows.  The launches need the run lengths on the host:
        // a copy of E + 1 integers and a wait, a few microseconds against the milliseconds of such a step.
        FT_CHECK_CUDA(cudaMemcpyAsync(L.h_seg, L.seg, (size_t)(c.experts + 1) * 4, cudaMemcpyDeviceToHost, st));
        if (scaled_in) FT_TRY(launch_scaled_rows(L.hn, L.wts, L.slot_pos, top, nullptr, L.mx_hi, L.mx_lo, pairs, W, st));
        else FT_TRY(launch_gather_planes_rows(L.hn, L.slot_token, L.mx_hi, L.mx_lo, pairs, W, st));
        FT_CHECK_CUDA(cudaStreamSynchronize(st));
        auto off = [](const void* p, size_t elems) { return (const void*)((const uint8_t*)p + elems * 2); };
        ft_gemm_epilogue ep = {};
        ep.mode = FT_EPI_PARTIAL;
        auto lane_of = [&](int k) { return k % (Layered::kSide + 1) == 0 ? st : L.side[k % (Layered::kSide + 1) - 1]; };
        auto join = [&]() -> int {          // the engine's stream waits for what the side streams were given
            for (int k = 0; k < Layered::kSide; ++k) {
                FT_CHECK_CUDA(cudaEventRecord(L.side_done[k], L.side[k]));
                FT_CHECK_CUDA(cudaStreamWaitEvent(st, L.side_done[k], 0));
            }
            return 0;
        };
        FT_CHECK_CUDA(cudaEventRecord(L.main_ready, st));
        for (int i = 0; i < Layered::kSide; ++i) FT_CHECK_CUDA(cudaStreamWaitEvent(L.side[i], L.main_ready, 0));
        int k = 0;
        for (int x = 0; x < c.experts; ++x) {
            const int r0 = L.h_seg[x], nr = L.h_seg[x + 1] - r0;
            if (nr <= 0) continue;
            ep.out = L.gu + (size_t)r0 * n_up;
            FT_TRY(ft_gemm_fused(off(c.w_gu, (size_t)x * n_up * W), off(L.mx_hi, (size_t)r0 * W),
                                 off(L.mx_lo, (size_t)r0 * W), n_up, nr, W, 1, &ep, lane_of(k++)));
            launched();
        }
        FT_TRY(join());
        FT_TRY(launch_swiglu_planes(L.gu, L.ax_hi, L.ax_lo, (size_t)pairs * c.ff, st, act));
        FT_CHECK_CUDA(cudaEventRecord(L.main_ready, st));
        for (int i = 0; i < Layered::kSide; ++i) FT_CHECK_CUDA(cudaStreamWaitEvent(L.side[i], L.main_ready, 0));
        k = 0;
        for (int x = 0; x < c.experts; ++x) {
            const int r0 = L.h_seg[x], nr = L.h_seg[x + 1] - r0;
            if (nr <= 0) continue;
            ep.out = L.eout + (size_t)r0 * W;
            FT_TRY(ft_gemm_fused(off(c.w_down, (size_t)x * W * c.ff), off(L.ax_hi, (size_t)r0 * c.ff),
                                 off(L.ax_lo, (size_t)r0 * c.ff), W, nr, c.ff, 1, &ep, lane_of(k++)));
            launched();
        }
        FT_TRY(join());
        launched(4);
    } else {
        LinearArgs gu;                  // first matrix of every (token, choice) pair, grouped by expert, with its activation
        gu.A = L.hn; gu.a_rows = L.slot_token; gu.lda = W; gu.W = (const __nv_bfloat16*)c.w_gu;
        if (scaled_in) {                // the scaled rows wait in L.eout, which the second matrix overwrites afterwards
            FT_TRY(launch_scaled_rows(L.hn, L.wts, L.slot_pos, top, L.eout, nullptr, nullptr, pairs, W, st));
            launched();
            gu.A = L.eout; gu.a_rows = nullptr;
        }
        gu.w_stride = (long long)n_up * W; gu.ldw = W; gu.C = L.act; gu.ldc = c.ff; gu.seg = L.seg;
        gu.N = n_up; gu.K = W; gu.P = c.experts; gu.epi = act == FT_ACT_SWIGLU ? LIN_SWIGLU_PAIR : LIN_RELU2;
        FT_TRY(launch_linear(gu, T * top, st));
        LinearArgs dn;
        dn.A = L.act; dn.lda = c.ff; dn.W = (const __nv_bfloat16*)c.w_down; dn.w_stride = (long long)W * c.ff;
        dn.ldw = c.ff; dn.C = L.eout; dn.ldc = W; dn.seg = L.seg; dn.N = W; dn.K = c.ff; dn.P = c.experts;
        FT_TRY(launch_linear(dn, T * top, st));
    }
    launched(4);
    return 0;
}

// out [T][width] = W_down act(W_up in) for every row: the dense feed-forward and the shared expert of a sandwich layer.
// `in` is the normed stream L.hn (hi / lo: its planes when the step has them).
static int run_mlp(Engine* e, const void* hi, const void* lo, const void* w_up, const void* w_down, int ff, int act, float* out,
                   int T) {
    Layered& L = *e->lay;
    const int W = L.m.width;
    const int n_up = act == FT_ACT_SWIGLU ? 2 * ff : ff;
    cudaStream_t st = e->stream;
    if (L.tensor && T >= kTensorMinRows && n_up % 128 == 0 && W % 64 == 0 && W % 128 == 0 && ff % 64 == 0) {
        FT_TRY(dense(e, L.hn, hi, lo, w_up, L.ffa, T, n_up, W));
        FT_TRY(launch_swiglu_planes(L.ffa, L.ax_hi, L.ax_lo, (size_t)T * ff, st, act));
        e->st.kernel_launches++;
        return dense(e, nullptr, L.ax_hi, L.ax_lo, w_down, out, T, W, ff);
    }
    LinearArgs up;
    up.A = L.hn; up.lda = W; up.W = (const __nv_bfloat16*)w_up; up.ldw = W; up.C = L.ffb; up.ldc = ff; up.M = T; up.N = n_up;
    up.K = W; up.epi = act == FT_ACT_SWIGLU ? LIN_SWIGLU_PAIR : LIN_RELU2;
    FT_TRY(launch_linear(up, T, st));
    e->st.kernel_launches++;
    return dense(e, L.ffb, nullptr, nullptr, w_down, out, T, W, ff);
}

// One branch of a branch mixer: from the layer's stacked projection L.proj to `y` [T][width] (before its out_scale).
static int run_branch(Engine* e, const Batch& b, const LayeredLayer& ll, int k, float* y) {
    Layered& L = *e->lay;
    const ft_layered_model& M = L.m;
    const ft_branch_desc& c = ll.d.branch[k];
    StepMeta& m = e->meta;
    int* d = m.d;
    const int T = b.T, ld = ll.d.n_in;
    cudaStream_t st = e->stream;
    auto launched = [&](int n = 1) { e->st.kernel_launches += n; };
    const float* fin = L.bfin;
    int fin_cols = c.heads * c.vdim;
    if (c.kind == FT_BRANCH_WINDOW_ATTENTION || c.kind == FT_BRANCH_LATENT_WINDOW) {
        WindowArgs a;
        a.q_out = L.bq; a.cache = L.kv_cache + ll.br_cache_off[k];
        a.positions = d + m.o_pos; a.seq_rows = d + m.o_rows; a.page_table = d + m.o_pt; a.max_pages = e->max_pages;
        a.rot_freq = c.rot_freq; a.rot_dims = c.rot_dims; a.window = c.window; a.scale = c.scale; a.softcap = c.softcap;
        a.out = L.bfin; a.H = c.heads;
        if (c.kind == FT_BRANCH_WINDOW_ATTENTION) {
            a.proj = L.proj; a.ldp = ld; a.o_q = c.o_q; a.o_k = c.o_k; a.o_v = c.o_v;
            a.q_gain = c.q_gain; a.k_gain = c.k_gain; a.rot_half = c.rot_half; a.rot_mag = c.rot_mag != 0.f ? c.rot_mag : 1.f;
            a.chunked = c.chunked;
            if (c.kv_lender > 0) {          // another layer's keys and values: it has written the step's rows already
                a.cache = L.kv_cache + L.layers[c.kv_lender - 1].br_cache_off[ll.lender_branch[k]];
                a.no_kv = 1;
            }
            if (c.conv >= 1) {
                // q | k | v through their short convolutions over time (no bias, no activation) into L.bv; the slot keeps the
                // last projected rows
                const int nq = c.heads * c.dim, nk = c.kv_lender > 0 ? 0 : c.kv_heads * c.dim, nv = c.kv_lender > 0 ? 0 : c.kv_heads * c.vdim;
                SpaceArgs s;
                s.proj = L.proj; s.ldp = ld; s.o_x = c.o_q; s.channels = nq + nk + nv; s.taps = c.conv; s.heads = 0; s.act = 0;
                s.conv_w = c.conv_w; s.xbc = L.bv; s.state = L.state; s.slot_stride = (long long)L.slot_stride;
                s.tail_off = (long long)ll.br_x_off[k];
                s.seq_rows = d + m.o_rows; s.req_start = d + m.o_xstart; s.req_pos0 = d + m.o_xpos0; s.req_slot = d + m.o_xslot;
                FT_TRY(launch_space_prep(s, T, b.n_req, st));
                launched(2);
                a.proj = L.bv; a.ldp = s.channels; a.o_q = 0; a.o_k = nq; a.o_v = nq + nk;
            }
            a.q_bias = c.q_bias; a.k_bias = c.k_bias;
            a.G = c.kv_heads; a.dim = c.dim; a.vdim = c.vdim;
            a.qk_norm = c.qk_norm; a.eps = M.eps; a.keep_first = c.keep_first; a.sink = c.sink; a.rel = c.rel; a.rel_n = c.rel_n;
            a.v_bias = c.v_bias; a.v_role = c.v_role; a.v_mix = c.v_mix; a.v_first = L.v_first;
        } else {
            // One shared key head: cached key [rotated part | normed latent], the value is its latent part.  The plain query
            // part is folded through W_uk into latent space, so no per-head key or value is ever formed.
            const int H = c.heads, R = c.rot_dims, C = c.kv_rank, D = c.dim, kd = R + C, ls = H * kd + kd;
            FT_TRY(launch_rms_cols(L.proj, ld, c.o_q, c.q_norm, L.b1, c.q_rank, 0, c.q_rank, M.eps, T, st));
            FT_TRY(dense(e, L.b1, nullptr, nullptr, c.w_uq, L.b2, T, H * (D + R), c.q_rank));
            FT_TRY(launch_latent_stage(L.b2, H, D, R, L.proj, ld, c.o_k, C, c.kv_norm, M.eps, L.lstage, ls, T, st));
            LinearArgs f;                   // q_lat_h = W_uk_h^T q_plain_h, beside the rotated part of head h
            f.A = L.b2; f.lda = H * (D + R); f.a_col_stride = D + R;
            f.W = (const __nv_bfloat16*)c.w_uk_t; f.w_stride = (long long)C * D; f.ldw = D;
            f.C = L.lstage + R; f.ldc = ls; f.c_col_stride = kd; f.M = T; f.N = C; f.K = D; f.P = H;
            FT_TRY(launch_linear(f, T, st));
            launched(3);
            a.proj = L.lstage; a.ldp = ls; a.o_q = 0; a.o_k = H * kd; a.o_v = -1; a.v_in_key = R;
            a.G = 1; a.dim = kd; a.vdim = C;
        }
        WindowTiles tm;
        tm.tile_req = d + m.o_treq; tm.tile_q0 = d + m.o_tq0; tm.req_q_start = d + m.o_qstart; tm.req_slot = d + m.o_rslot;
        tm.req_pos0 = d + m.o_rpos0; tm.n_tiles = b.n_tiles;
        FT_TRY(launch_window_attention(a, T, b.n_decode, tm, st));
        launched(b.n_tiles > 0 && b.n_decode > 0 ? 3 : 2);
        if (c.kind == FT_BRANCH_LATENT_WINDOW) {
            LinearArgs v;                   // values out of latent space: o_h = W_uv_h (sum_j p_j c_j)
            v.A = L.bfin; v.lda = c.heads * c.kv_rank; v.a_col_stride = c.kv_rank;
            v.W = (const __nv_bfloat16*)c.w_uv; v.w_stride = (long long)c.vdim * c.kv_rank; v.ldw = c.kv_rank;
            v.C = L.b3; v.ldc = c.heads * c.vdim; v.c_col_stride = c.vdim;
            v.M = T; v.N = c.vdim; v.K = c.kv_rank; v.P = c.heads;
            FT_TRY(launch_linear(v, T, st));
            launched();
            fin = L.b3;
        }
    } else if (c.kind == FT_BRANCH_SELECTIVE_SCAN) {
        // x through its convolution (bias, SiLU) -> (low | B | C) = W_x x -> dt_raw = W_dt low -> the scan, gated by silu(z)
        const int inner = c.heads, N = c.dim, R = c.dt_rank, nl = c.x_rows > 0 ? c.x_rows : R + 2 * N;
        const int kdt = c.x_rows > 0 ? c.x_rows : R;       // columns of w_dt
        SpaceArgs s;
        s.proj = L.proj; s.ldp = ld; s.o_x = c.o_v; s.channels = inner; s.taps = c.conv; s.heads = 0; s.act = 1;
        s.conv_w = c.conv_w; s.conv_b = c.conv_b; s.xbc = L.bv; s.state = L.state; s.slot_stride = (long long)L.slot_stride;
        s.tail_off = (long long)ll.br_x_off[k];
        s.seq_rows = d + m.o_rows; s.req_start = d + m.o_xstart; s.req_pos0 = d + m.o_xpos0; s.req_slot = d + m.o_xslot;
        FT_TRY(launch_space_prep(s, T, b.n_req, st));
        launched(2);
        FT_TRY(dense(e, L.bv, nullptr, nullptr, c.w_x, L.b1, T, nl, inner));
        // the step sizes' pre-activation from the first R columns of the low-rank row (the whole row when w_dt is padded)
        if (kdt == nl) {
            FT_TRY(dense(e, L.b1, nullptr, nullptr, c.w_dt, L.b2, T, inner, nl));
        } else {
            LinearArgs dtp;
            dtp.A = L.b1; dtp.lda = nl; dtp.W = (const __nv_bfloat16*)c.w_dt; dtp.ldw = kdt; dtp.C = L.b2; dtp.ldc = inner;
            dtp.M = T; dtp.N = inner; dtp.K = kdt;
            FT_TRY(launch_linear(dtp, T, st));
        }
        ScanArgs sc;
        sc.x = L.bv; sc.ldx = inner; sc.dt_raw = L.b2; sc.ldd = inner; sc.B = L.b1 + R; sc.C = L.b1 + R + N; sc.ldbc = nl;
        sc.z = L.proj + c.o_z; sc.ldz = ld; sc.dt_bias = c.dt_bias; sc.a_log = c.a_log; sc.skip = c.skip; sc.out = L.bfin;
        sc.state = L.state; sc.slot_stride = (long long)L.slot_stride; sc.s_off = (long long)ll.br_s_off[k];
        sc.req_start = d + m.o_xstart; sc.req_pos0 = d + m.o_xpos0; sc.req_slot = d + m.o_xslot;
        sc.channels = inner; sc.N = N; sc.rows = T; sc.ws = L.scan_ws; sc.ws_rows = L.scan_ws_rows;
        FT_TRY(launch_selective_scan(sc, b.n_req, st));
        launched(2);
    } else {
        RecurArgs r;
        r.ab = L.ab; r.o = L.bo; r.state = L.state; r.slot_stride = (long long)L.slot_stride; r.s_off = (long long)ll.br_s_off[k];
        r.req_start = d + m.o_xstart; r.req_pos0 = d + m.o_xpos0; r.req_slot = d + m.o_xslot;
        r.heads = c.heads; r.qk_heads = c.kv_heads; r.dim = c.dim; r.vd = c.vdim; r.ldo = c.heads * c.vdim;
        ReadoutArgs o;
        o.o = L.bo; o.vd = c.vdim; o.vdim = c.vdim; o.heads = c.heads; o.gain = c.out_norm; o.eps = M.eps; o.out = L.bfin;
        if (c.kind == FT_BRANCH_DECAY_ATTENTION) {
            // q | k | v are adjacent columns of the projection: SiLU in place, then the rule reads them where they are
            FT_TRY(launch_silu_cols(L.proj, ld, c.o_q, 2 * c.kv_heads * c.dim + c.heads * c.vdim, T, st));
            FT_TRY(launch_const_decay(c.decay, L.ab, c.heads, T, st));
            r.q = L.proj + c.o_q; r.k = L.proj + c.o_k; r.v = L.proj + c.o_v; r.ldq = r.ldk = r.ldv = ld;
            o.gate = L.proj + c.o_g; o.ldg = ld; o.gate_kind = 2; o.norm_groups = 1;
            launched(2);
        } else if (c.kind == FT_BRANCH_MATRIX_MEMORY) {
            MemoryArgs g;
            g.proj = L.proj; g.ldp = ld; g.o_v = c.o_v; g.o_i = c.o_i; g.o_f = c.o_f; g.gate_bias = c.gate_bias; g.cap = c.gate_cap;
            g.heads = c.heads; g.vdim = c.vdim; g.v_ext = L.bv; g.gates = L.gates; g.ab = L.ab; g.floor = L.floor;
            g.state = L.state; g.slot_stride = (long long)L.slot_stride; g.m_off = (long long)ll.br_x_off[k];
            g.req_start = r.req_start; g.req_pos0 = r.req_pos0; g.req_slot = r.req_slot;
            FT_TRY(launch_memory_prep(g, T, b.n_req, st));
            r.q = L.proj + c.o_q; r.k = L.proj + c.o_k; r.ldq = r.ldk = ld;
            r.v = L.bv; r.vd = c.vdim + 1; r.ldv = r.ldo = c.heads * (c.vdim + 1);
            o.vd = c.vdim + 1; o.q_scale = 1.f / sqrtf((float)c.dim); o.floor = L.floor;
            o.gate = L.proj + c.o_g; o.ldg = ld; o.gate_kind = 2; o.norm_groups = c.heads;
            launched(2);
        } else {
            const int inner = c.heads * c.vdim, gn = c.kv_heads * c.dim;
            SpaceArgs s;
            s.proj = L.proj; s.ldp = ld; s.o_x = c.o_v; s.o_dt = c.o_dt; s.channels = inner + 2 * gn; s.taps = c.conv;
            s.heads = c.heads; s.conv_w = c.conv_w; s.conv_b = c.conv_b; s.dt_bias = c.dt_bias; s.a_log = c.a_log;
            s.xbc = L.bv; s.ab = L.ab; s.state = L.state; s.slot_stride = (long long)L.slot_stride;
            s.tail_off = (long long)ll.br_x_off[k];
            s.seq_rows = d + m.o_rows; s.req_start = r.req_start; s.req_pos0 = r.req_pos0; s.req_slot = r.req_slot;
            FT_TRY(launch_space_prep(s, T, b.n_req, st));
            r.v = L.bv; r.k = L.bv + inner; r.q = L.bv + inner + gn; r.ldq = r.ldk = r.ldv = s.channels;
            o.skip = c.skip; o.x = L.bv; o.ldx = s.channels;
            o.gate = L.proj + c.o_z; o.ldg = ld; o.gate_kind = 1; o.norm_groups = c.norm_groups;
            launched(2);
        }
        o.ldo = r.ldo;
        FT_TRY(launch_decay_rule(r, b.n_req, T, st));
        FT_TRY(launch_readout(o, T, st));
        launched(2);
    }
    return dense(e, fin, nullptr, nullptr, c.w_o, y, T, M.width, fin_cols);
}

// Forward pass of a layered model.  Per layer: ONE projection of the normed input into all the parts that read it
// (queries, latents or q/k/v, gates, low-rank inner products, residual gates, router logits), the mixer, the feed-forward, and
// one kernel per sublayer joint that updates the residual stream and norms it for what reads it next.
static int forward_layered(Engine* e, const Batch& b) {
    Layered& L = *e->lay;
    const ft_layered_model& M = L.m;
    StepMeta& m = e->meta;
    int* d = m.d;
    const int T = b.T, W = M.width;
    cudaStream_t st = e->stream;
    void* hn_hi = L.tensor && T >= kTensorMinRows ? L.hn_hi : nullptr;      // planes of the normed input, written by its producer
    void* hn_lo = hn_hi ? L.hn_lo : nullptr;
    auto launched = [&](int n = 1) { e->st.kernel_launches += n; };
    const int n_streams = std::max(M.streams, 1);
    const bool trail = L.trail_on && L.trail;
    auto hyper_next = [&](HyperArgs& h, const float* in_next, const float* nw, const float* nb) {
        h.X = L.streams; h.S = n_streams; h.W = W; h.eps = M.eps;
        h.in_next = in_next; h.nw = nw; h.nb = nb; h.hn = L.hn; h.hi = hn_hi; h.lo = hn_lo;
    };
    if (L.hyper) {
        HyperArgs h;
        const ft_layer_desc& c0 = L.layers[0].d;
        hyper_next(h, c0.hc_in[0], c0.norm_pre1, c0.norm_pre1_b);
        h.tokens = d + m.o_tokens; h.embed = M.embed; h.embed_scale = M.embed_scale != 0.f ? M.embed_scale : 1.f;
        FT_TRY(launch_hyper_joint(h, T, st));
    } else if (L.postnorm)
        FT_TRY(launch_embed_scale(d + m.o_tokens, M.embed, M.embed_scale != 0.f ? M.embed_scale : 1.f, e->resid, L.hist, T, W, st));
    else
        FT_TRY(launch_embed_norm(d + m.o_tokens, M.embed, e->resid, L.hn, hn_hi, hn_lo, T, W, M.eps, L.layers[0].d.norm_gain,
                                 L.layers[0].d.form == FT_LAYER_SANDWICH ? L.layers[0].d.norm_pre1 : nullptr, st));
    launched();
    // what the mixer of a post-norm layer reads: the stream plus its short convolution over time
    auto canon = [&](const LayeredLayer& ll) -> int {
        const ft_layer_desc& c = ll.d;
        CanonArgs ca;
        ca.x = e->resid; ca.hn = L.hn; ca.hi = hn_hi; ca.lo = hn_lo; ca.W = W;
        ca.w = c.canon_taps >= 1 ? c.canon1 : nullptr; ca.taps = c.canon_taps;
        ca.state = L.state; ca.slot_stride = (long long)L.slot_stride; ca.tail_off = (long long)ll.canon_off[0];
        ca.seq_rows = d + m.o_rows; ca.req_start = d + m.o_xstart; ca.req_pos0 = d + m.o_xpos0; ca.req_slot = d + m.o_xslot;
        FT_TRY(launch_canon(ca, T, st));
        launched();
        return 0;
    };
    for (int l = 0; l < M.n_layers; ++l) {
        const LayeredLayer& ll = L.layers[l];
        const ft_layer_desc& c = ll.d;
        const bool sandwich = c.form == FT_LAYER_SANDWICH;
        const int ld = c.n_in;              // row stride of this layer's projection outputs
        if (c.form == FT_LAYER_POSTNORM) FT_TRY(canon(ll));
        FT_TRY(dense(e, L.hn, hn_hi, hn_lo, c.w_in, L.proj, T, c.n_in, W));
        const float *y0 = L.mix, *y1 = nullptr;      // the mixer's result: s0 * y0 + s1 * y1, each [T][width]
        float s0 = 1.f, s1 = 1.f;
        if (c.mixer == FT_MIXER_BRANCHES) {
            FT_TRY(run_branch(e, b, ll, 0, L.mix));
            s0 = c.branch[0].out_scale;
            if (c.n_branches > 1) {
                FT_TRY(run_branch(e, b, ll, 1, L.mix2));
                y1 = L.mix2;
                s1 = c.branch[1].out_scale;
            }
        } else {
        const float* mixed = nullptr;      // [T][heads * vdim], input of the output projection
        if (c.mixer == FT_MIXER_LATENT_ATTENTION) {
            float* cache = L.lat_cache + ll.cache_off;
            void* cache16 = L.lat_cache16 ? (uint8_t*)L.lat_cache16 + ll.cache_off * 2 : nullptr;
            FT_TRY(launch_latent_write(L.proj, ld, c.o_dkv, c.dkv_norm, cache, cache16, d + m.o_pos, d + m.o_rows, d + m.o_pt,
                                       e->max_pages, c.kv_rank, M.eps, T, st));
            LinearArgs a;                   // queries into latent space, head by head: qlat_h = W_uk_h^T q_h
            a.A = L.proj + c.o_q; a.lda = ld; a.a_col_stride = c.dim;
            a.W = (const __nv_bfloat16*)c.w_uk_t; a.w_stride = (long long)c.kv_rank * c.dim; a.ldw = c.dim;
            a.C = L.b1; a.ldc = c.heads * c.kv_rank; a.c_col_stride = c.kv_rank;
            a.M = T; a.N = c.kv_rank; a.K = c.dim; a.P = c.heads;
            FT_TRY(launch_linear(a, T, st));
            FT_TRY(launch_latent_attn(L.b1, cache, cache16, L.proj, ld, c.o_gate, L.b2, L.attn_part, d + m.o_pos, d + m.o_rows, d + m.o_pt,
                                      e->max_pages, c.heads, c.kv_rank, c.scale, T, st));
            LinearArgs v;                   // values out of latent space: o_h = W_uv_h (sum_j p_j c_j)
            v.A = L.b2; v.lda = c.heads * c.kv_rank; v.a_col_stride = c.kv_rank;
            v.W = (const __nv_bfloat16*)c.w_uv; v.w_stride = (long long)c.vdim * c.kv_rank; v.ldw = c.kv_rank;
            v.C = L.b3; v.ldc = c.heads * c.vdim; v.c_col_stride = c.vdim;
            v.M = T; v.N = c.vdim; v.K = c.kv_rank; v.P = c.heads;
            FT_TRY(launch_linear(v, T, st));
            launched(4);
            mixed = L.b3;
        } else {
            DeltaArgs da;
            const float* gate = L.proj + c.o_g1;
            int ldg = ld;
            if (c.rank_a > 0) {             // second halves of the low-rank decay and gate projections
                LinearArgs a;
                a.A = L.proj + c.o_a1; a.lda = ld; a.W = (const __nv_bfloat16*)c.w_a2; a.ldw = c.rank_a;
                a.C = L.b1; a.ldc = c.heads * c.dim; a.M = T; a.N = c.heads * c.dim; a.K = c.rank_a;
                FT_TRY(launch_linear(a, T, st));
                da.araw = L.b1;
            } else {                        // one decay per head and token, straight from the stacked projection
                da.araw = L.proj + c.o_a1; da.head_decay = 1; da.ld_araw = ld;
            }
            if (c.rank_g > 0) {
                LinearArgs g;
                g.A = L.proj + c.o_g1; g.lda = ld; g.W = (const __nv_bfloat16*)c.w_g2; g.ldw = c.rank_g;
                g.C = L.b2; g.ldc = c.heads * c.vdim; g.M = T; g.N = c.heads * c.vdim; g.K = c.rank_g;
                FT_TRY(launch_linear(g, T, st));
                gate = L.b2; ldg = 0;
            }
            da.proj = L.proj; da.ldp = ld; da.o_q = c.o_q; da.o_beta = c.o_beta;
            da.conv = c.conv_w; da.dt_bias = c.dt_bias; da.a_log = c.a_log;
            da.qkv = L.b3; da.decay = L.b1; da.beta = L.beta; da.o = L.b4;
            da.state = L.state; da.slot_stride = (long long)L.slot_stride; da.s_off = (long long)ll.s_off;
            da.tail_off = (long long)ll.tail_off;
            da.seq_rows = d + m.o_rows; da.req_start = d + m.o_xstart; da.req_pos0 = d + m.o_xpos0;
            da.req_slot = d + m.o_xslot;
            da.heads = c.heads; da.kvh = c.kv_heads; da.dim = c.dim; da.vdim = c.vdim; da.taps = c.conv;
            FT_TRY(launch_delta(da, gate, c.out_norm, M.eps, T, b.n_req, st, ldg, c.gate_act));
            launched(6);
            mixed = L.b4;
        }
        FT_TRY(dense(e, mixed, nullptr, nullptr, c.w_o, L.mix, T, W, c.heads * c.vdim));
        }
        const ft_layer_desc* nx = l + 1 < M.n_layers ? &L.layers[l + 1].d : nullptr;
        // gains of the norm that the next layer (or the head) reads: one number, or one per coordinate
        const float gain_next = nx ? nx->norm_gain : M.final_norm_gain;
        const float* gain_next_w = nx ? (nx->form == FT_LAYER_SANDWICH ? nx->norm_pre1 : nullptr) : M.final_norm_w;
        if (c.form == FT_LAYER_HYPER) {
            // every stream is rebuilt from the old ones and the sublayer's result; the same kernel forms what reads them next
            const bool has_ff = c.ff_kind != FT_FF_NONE;
            const float* in_after = nx ? nx->hc_in[0] : nullptr;          // the head reads the plain sum
            const float* nw_after = nx ? nx->norm_pre1 : M.final_norm_w;
            const float* nb_after = nx ? nx->norm_pre1_b : M.final_norm_b;
            HyperArgs h1;
            if (has_ff) hyper_next(h1, c.hc_in[1], c.norm_pre2, c.norm_pre2_b);
            else hyper_next(h1, in_after, nw_after, nb_after);
            h1.y0 = y0; h1.y1 = y1; h1.s0 = s0; h1.s1 = s1; h1.mix = c.hc_mix[0]; h1.out = c.hc_out[0];
            if (c.mixer == FT_MIXER_BRANCHES) { h1.g0 = c.branch[0].out_gain; h1.g1 = y1 ? c.branch[1].out_gain : nullptr; }
            if (!has_ff && trail) h1.sum_out = e->resid;
            FT_TRY(launch_hyper_joint(h1, T, st));
            launched();
            if (has_ff) {
                HyperArgs h2;
                hyper_next(h2, in_after, nw_after, nb_after);
                h2.mix = c.hc_mix[1]; h2.out = c.hc_out[1];
                if (c.ff_kind == FT_FF_DENSE) {
                    FT_TRY(run_mlp(e, hn_hi, hn_lo, c.w_gu, c.w_down, c.ff, c.ff_act, L.mix, T));
                    h2.y0 = L.mix;
                } else {
                    const int ldl = c.router_rows > 0 ? c.router_rows : c.experts;
                    FT_TRY(dense(e, L.hn, hn_hi, hn_lo, c.w_router, L.rlog, T, ldl, W));
                    FT_TRY(run_experts(e, c, L.rlog, ldl, 0, T));
                    h2.eout = L.eout; h2.slot_pos = L.slot_pos; h2.top = c.top;
                    h2.wt = c.route_input ? nullptr : L.wts;
                    if (c.shared_ff > 0) {
                        FT_TRY(run_mlp(e, hn_hi, hn_lo, c.w_shared_up, c.w_shared_down, c.shared_ff, c.ff_act, L.mix, T));
                        h2.y0 = L.mix;
                    }
                }
                if (trail) h2.sum_out = e->resid;
                FT_TRY(launch_hyper_joint(h2, T, st));
                launched();
            }
        } else if (c.form == FT_LAYER_POSTNORM) {
            // x += norm(mixer);  x += norm(ff(x + conv(x)));  the layer's result joins the depth history and the stream that
            // goes on is the weighted sum over it
            // One kernel per joint: it also keeps the rows the sublayer read for the next step's convolution and forms what
            // reads the stream next (the feed-forward's input, or the sum over depth).
            const bool has_ff = c.ff_kind != FT_FF_NONE;
            // In the fused form a row's CTA forms its taps - 1 predecessors again; that pays while launches, not bytes, bound
            // the step.  Both forms add the same numbers in the same order.
            const bool fuse_next = c.canon_taps >= 1 && T <= kFuseCanonRows;
            auto joint = [&](PostNormArgs& p, int which) {
                p.W = W; p.eps = M.eps; p.taps = c.canon_taps;
                p.state = L.state; p.slot_stride = (long long)L.slot_stride;
                p.save_off = c.canon_taps > 1 ? (long long)ll.canon_off[which] : -1;
                p.seq_rows = d + m.o_rows; p.req_start = d + m.o_xstart; p.req_pos0 = d + m.o_xpos0; p.req_slot = d + m.o_xslot;
            };
            auto ends_layer = [&](PostNormArgs& p) { p.x_out = e->resid; p.hist = L.hist; p.depth_w = c.depth_w; p.k = l + 1; p.t_stride = e->t_max; };
            PostNormArgs pa;
            joint(pa, 0);
            pa.x = e->resid; pa.y0 = y0; pa.y1 = y1; pa.s0 = s0; pa.s1 = s1; pa.post_w = c.norm_post1;
            if (c.mixer == FT_MIXER_BRANCHES) { pa.b0 = c.branch[0].o_bias; pa.b1 = y1 ? c.branch[1].o_bias : nullptr; }
            if (!has_ff) {
                ends_layer(pa);
            } else if (fuse_next) {              // the feed-forward's input in the same pass
                pa.x_out = L.resid2; pa.cw = c.canon2; pa.read_off = (long long)ll.canon_off[1];
                pa.hn = L.hn; pa.hi = hn_hi; pa.lo = hn_lo;
            } else {
                pa.x_out = L.resid2;
            }
            FT_TRY(launch_postnorm(pa, T, st));
            launched();
            if (has_ff) {
                if (!fuse_next) {                 // the feed-forward's input in a pass of its own
                    CanonArgs ca;
                    ca.x = L.resid2; ca.hn = L.hn; ca.hi = hn_hi; ca.lo = hn_lo; ca.W = W;
                    ca.w = c.canon_taps >= 1 ? c.canon2 : nullptr; ca.taps = c.canon_taps;
                    ca.state = L.state; ca.slot_stride = (long long)L.slot_stride; ca.tail_off = (long long)ll.canon_off[1];
                    ca.seq_rows = d + m.o_rows; ca.req_start = d + m.o_xstart; ca.req_pos0 = d + m.o_xpos0; ca.req_slot = d + m.o_xslot;
                    FT_TRY(launch_canon(ca, T, st));
                    launched();
                }
                FT_TRY(run_mlp(e, hn_hi, hn_lo, c.w_gu, c.w_down, c.ff, c.ff_act, L.mix, T));
                PostNormArgs pf;
                joint(pf, 1);
                pf.x = L.resid2; pf.y0 = L.mix; pf.post_w = c.norm_post2;
                ends_layer(pf);
                FT_TRY(launch_postnorm(pf, T, st));
                launched();
            }
        } else if (sandwich) {
            FT_REQUIRE(gain_next_w, "engine: layer %d: a sandwich layer needs per-coordinate gains in what follows it", l);
            SandwichArgs sa;
            sa.x = e->resid; sa.hn = L.hn; sa.hi = hn_hi; sa.lo = hn_lo; sa.W = W; sa.eps = M.eps;
            sa.y0 = y0; sa.s0 = s0; sa.y1 = y1; sa.s1 = s1; sa.post_w = c.norm_post1;
            sa.next_w = c.ff_kind != FT_FF_NONE ? c.norm_pre2 : gain_next_w;
            FT_TRY(launch_sandwich_norm(sa, T, st));
            launched();
            if (c.ff_kind != FT_FF_NONE) {
                SandwichArgs sf;
                sf.x = e->resid; sf.hn = L.hn; sf.hi = hn_hi; sf.lo = hn_lo; sf.W = W; sf.eps = M.eps;
                sf.post_w = c.norm_post2; sf.next_w = gain_next_w;
                if (c.ff_kind == FT_FF_DENSE) {
                    FT_TRY(run_mlp(e, hn_hi, hn_lo, c.w_gu, c.w_down, c.ff, c.ff_act, L.mix, T));
                    sf.y0 = L.mix;
                } else {
                    // router logits: fp32 accumulation over fp32 activations (CUDA cores), or over their bf16 hi + lo planes
                    // on the tensor cores when the step is large; the router's rows are padded to whole tiles for that
                    const int ldl = c.router_rows > 0 ? c.router_rows : c.experts;
                    FT_TRY(dense(e, L.hn, hn_hi, hn_lo, c.w_router, L.rlog, T, ldl, W));
                    FT_TRY(run_experts(e, c, L.rlog, ldl, 0, T));
                    sf.eout = L.eout; sf.wt = L.wts; sf.slot_pos = L.slot_pos; sf.top = c.top;
                    if (c.shared_ff > 0) {
                        FT_TRY(run_mlp(e, hn_hi, hn_lo, c.w_shared_up, c.w_shared_down, c.shared_ff, c.ff_act, L.mix, T));
                        sf.y0 = L.mix;
                    }
                }
                FT_TRY(launch_sandwich_norm(sf, T, st));
                launched();
            }
        } else {
            int top = 0;
            if (c.ff_kind == FT_FF_MOE) {
                top = c.top;
                FT_TRY(run_experts(e, c, L.proj, ld, c.o_router, T));
            }
            FT_REQUIRE(!gain_next_w, "engine: layer %d: a gated layer is followed by a norm with one gain", l);
            FT_TRY(launch_combine_norm(e->resid, L.hn, L.proj, ld, c.o_rg1, c.o_rg2, c.rg_bias, L.mix, L.eout, L.wts,
                                       L.slot_pos, top, T, W, M.eps, gain_next, hn_hi, hn_lo, st));
            launched();
        }
        if (L.trail_on && L.trail)
            FT_CHECK_CUDA(cudaMemcpyAsync(L.trail + (size_t)l * e->t_max * W, e->resid, (size_t)T * W * 4,
                                          cudaMemcpyDeviceToDevice, st));
    }
    if (b.n_logit_rows > 0 && L.postnorm && !L.hyper) {
        // the model's norm over the wanted rows only, then the head
        FT_TRY(launch_rms_rows(e->resid, b.logit_rows_identity ? nullptr : d + m.o_lrow, M.final_norm_w, M.final_norm_gain, L.xlast,
                               b.n_logit_rows, W, M.eps, st));
        launched();
        FT_TRY(dense(e, L.xlast, nullptr, nullptr, M.head, e->logits, b.n_logit_rows, M.vocab, W, M.logit_softcap));
    } else if (b.n_logit_rows > 0) {
        const float* x = L.hn;
        if (!b.logit_rows_identity) {
            FT_TRY(launch_gather_rows(L.hn, d + m.o_lrow, L.xlast, b.n_logit_rows, W, st));
            launched();
            x = L.xlast;
        }
        FT_TRY(dense(e, x, nullptr, nullptr, M.head, e->logits, b.n_logit_rows, M.vocab, W, M.logit_softcap));
    }
    return 0;
}

static int upload_meta(Engine* e) {
    FT_CHECK_CUDA(cudaMemcpyAsync(e->meta.d, e->meta.h, e->meta.upload_ints * sizeof(int),
                                  cudaMemcpyHostToDevice, e->stream));
    e->st.h2d_bytes += (long long)(e->meta.upload_ints * sizeof(int));
    return 0;
}

static unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// ------------------------------------------------------------------ batch builder
// What a step runs for one sequence: its next `n` tokens, the first of them at position pos0.
struct Portion { Session* sess; const int* toks; int n; int pos0; };

// Fills the step's metadata block: decode rows (one token each) first, then prompt portions.  Shared by the scheduler's
// steps, ft_engine_feed and the debug hooks, so every path lays a batch out the same way.  Returns the summed context
// lengths of the decode rows.
static long long fill_batch(Engine* e, const std::vector<Portion>& dec, const std::vector<Portion>& pre, Batch& b) {
    StepMeta& m = e->meta;
    int* h = m.h;
    b.n_decode = (int)dec.size();
    b.n_prefill_req = (int)pre.size();
    b.n_req = b.n_decode + b.n_prefill_req;
    {
        int total = b.n_decode;
        for (const Portion& p : pre) total += p.n;
        layout_step(m, b.n_req, e->max_pages, total);
    }
    int row = 0;
    long long ctx_sum = 0;
    for (int i = 0; i < b.n_decode; ++i, ++row) {
        const Portion& p = dec[i];
        h[m.o_tokens + row] = p.toks[0];
        h[m.o_pos + row] = p.pos0;
        h[m.o_rows + row] = i;
        h[m.o_ctx + i] = p.pos0 + 1;
        ctx_sum += p.pos0 + 1;
        for (size_t k = 0; k < p.sess->pages.size(); ++k) h[m.o_pt + (size_t)i * e->max_pages + k] = p.sess->pages[k];
        h[m.o_xstart + i] = row;
        h[m.o_xpos0 + i] = p.pos0;
        h[m.o_xslot + i] = p.sess->slot;
    }
    int tiles = 0;
    h[m.o_qstart] = row;
    for (int j = 0; j < b.n_prefill_req; ++j) {
        const Portion& p = pre[j];
        const int pt_row = b.n_decode + j;
        h[m.o_xstart + pt_row] = row;
        h[m.o_xpos0 + pt_row] = p.pos0;
        h[m.o_xslot + pt_row] = p.sess->slot;
        for (int k = 0; k < p.n; ++k, ++row) {
            h[m.o_tokens + row] = p.toks[k];
            h[m.o_pos + row] = p.pos0 + k;
            h[m.o_rows + row] = pt_row;
        }
        h[m.o_qstart + j + 1] = row;
        h[m.o_rslot + j] = pt_row;
        h[m.o_rpos0 + j] = p.pos0;
        for (size_t k = 0; k < p.sess->pages.size(); ++k)
            h[m.o_pt + (size_t)pt_row * e->max_pages + k] = p.sess->pages[k];
        for (int q0 = 0; q0 < p.n; q0 += 64, ++tiles) {
            h[m.o_treq + tiles] = j;
            h[m.o_tq0 + tiles] = q0;
        }
    }
    h[m.o_xstart + b.n_req] = row;
    b.T = row;
    b.n_tiles = tiles;
    return ctx_sum;
}

// ------------------------------------------------------------------ one scheduler step
static int engine_step(Engine* e, std::unique_lock<std::mutex>& lk) {
    const ft_engine_config& c = e->cfg;
    StepMeta& m = e->meta;
    const auto t_begin = std::chrono::steady_clock::now();

    // retire finished requests from the active list
    e->active.erase(std::remove_if(e->active.begin(), e->active.end(),
                                   [&](Request* r) { return r->state == REQ_DONE; }),
                    e->active.end());
    // admit
    while (!e->waiting.empty() && (int)e->active.size() < c.max_batch) {
        Request* r = e->waiting.front();
        if (r->state == REQ_DONE) { e->waiting.pop_front(); continue; }
        if (!ensure_pages(e, r->sess, (int)r->prompt.size() + 1)) {
            if (e->active.empty()) {            // nothing will ever free pages for it
                e->waiting.pop_front();
                finish_request(e, r, 4, -1);
                continue;
            }
            break;
        }
        e->waiting.pop_front();
        r->state = REQ_PREFILL;
        e->active.push_back(r);
    }
    if (e->active.empty()) return 0;

    // ---- build the batch: decode rows first, then prefill chunks up to the token budget
    Batch b;
    int* h = m.h;
    std::vector<Request*> dec, pre;
    std::vector<int> pre_len;
    for (Request* r : e->active)
        if (r->state == REQ_DECODE) dec.push_back(r);
    int budget = c.max_batched_tokens - (int)dec.size();
    // Sessions that are streaming wait for the whole step: beside decode rows a step admits about
    // `decode_prefill_cap` prompt tokens (a ~1k-token chunk adds a few ms to a 1B step instead of the ~20 ms a full
    // 8192-token budget costs).  Once more than two sessions wait for their first token PER streaming session the
    // allowance grows in that proportion (cap x waiting / (2 x streaming)): a burst of 63 arrivals behind one early
    // bird gets the whole budget (one session waits 20 ms, 63 get their first token soonest), 56 arrivals beside 8
    // streaming sessions 3.5 x the cap, 35 beside 29 the cap — no cliff at "more waiting than streaming" that would
    // stall half of the sessions for a full-budget step.
    int n_pending = 0;
    for (Request* r : e->active) n_pending += r->state == REQ_PREFILL;
    if (e->decode_prefill_cap > 0 && !dec.empty()) {
        const long long n_dec = (long long)dec.size();
        const long long allow = (long long)e->decode_prefill_cap * std::max<long long>(n_pending, 2 * n_dec) / (2 * n_dec);
        // the projections work on 128-token tiles, so the rows up to the next tile boundary ride for free
        const long long rows = n_dec + allow;
        const long long tiled = (rows + kGemmTokenTile - 1) / kGemmTokenTile * kGemmTokenTile - n_dec;
        budget = (int)std::min<long long>(budget, tiled);
    }
    for (Request* r : e->active) {
        if (r->state != REQ_PREFILL || budget <= 0) continue;
        const int remaining = (int)r->prompt.size() - r->prefill_pos;
        const int take = std::min(remaining, budget);
        pre.push_back(r);
        pre_len.push_back(take);
        budget -= take;
    }
    // page growth for decode rows (evicting idle sessions if needed)
    for (size_t i = 0; i < dec.size();) {
        Request* r = dec[i];
        if (!ensure_pages(e, r->sess, (int)r->sess->tokens.size() + 1)) {
            finish_request(e, r, 2, -1);
            dec.erase(dec.begin() + i);
        } else {
            ++i;
        }
    }
    if (dec.empty() && pre.empty()) return 0;
    std::vector<Portion> dec_p, pre_p;
    for (Request* r : dec) dec_p.push_back({r->sess, &r->last_token, 1, (int)r->sess->tokens.size()});
    for (size_t j = 0; j < pre.size(); ++j)
        pre_p.push_back({pre[j]->sess, pre[j]->prompt.data() + pre[j]->prefill_pos, pre_len[j], pre[j]->prefill_pos});
    const long long ctx_sum = fill_batch(e, dec_p, pre_p, b);
    e->prof_ctx_sum = ctx_sum;
    e->st.decode_ctx_tokens += ctx_sum;
    // rows whose logits are sampled: every decode row, and the last row of a prompt that is complete
    int lrow = 0;
    for (int i = 0; i < b.n_decode; ++i) {
        h[m.o_lrow + lrow] = i;
        dec[i]->logits_row = lrow++;
    }
    for (int j = 0; j < b.n_prefill_req; ++j) {
        Request* r = pre[j];
        r->logits_row = -1;
        if (r->prefill_pos + pre_len[j] == (int)r->prompt.size()) {
            h[m.o_lrow + lrow] = h[m.o_qstart + j + 1] - 1;
            r->logits_row = lrow++;
        }
    }
    b.n_logit_rows = lrow;
    b.logit_rows_identity = lrow == b.T && b.n_prefill_req == 0;      // pure decode: row i wants logits row i
    // sampling parameters per logit row
    float* hf = reinterpret_cast<float*>(h);
    unsigned long long* hseed = reinterpret_cast<unsigned long long*>(h + m.o_seed);
    auto put_sampling = [&](Request* r) {
        const int lr = r->logits_row;
        hf[m.o_temp + lr] = r->temperature;
        h[m.o_topk + lr] = r->top_k;
        hf[m.o_topp + lr] = r->top_p;
        hseed[lr] = mix64(r->seed * 0x100000001B3ull + (unsigned long long)r->n_generated);
    };
    for (Request* r : dec) put_sampling(r);
    for (Request* r : pre) if (r->logits_row >= 0) put_sampling(r);

    e->prof_used = 0;
    FT_CHECK_CUDA(cudaEventRecord(e->s0, e->stream));
    FT_TRY(upload_meta(e));
    FT_TRY(forward(e, b));
    if (b.n_logit_rows > 0) {
        const float* dtemp = reinterpret_cast<const float*>(m.d + m.o_temp);
        const float* dtopp = reinterpret_cast<const float*>(m.d + m.o_topp);
        const unsigned long long* dseed = reinterpret_cast<const unsigned long long*>(m.d + m.o_seed);
        FT_TRY(launch_sample(e->logits, b.n_logit_rows, c.vocab, dtemp, m.d + m.o_topk, dtopp, dseed,
                             m.d + m.o_sampled, e->pdl, e->stream));
        e->st.kernel_launches++;
        FT_CHECK_CUDA(cudaMemcpyAsync(h + m.o_sampled, m.d + m.o_sampled, b.n_logit_rows * sizeof(int),
                                      cudaMemcpyDeviceToHost, e->stream));
    }
    FT_CHECK_CUDA(cudaEventRecord(e->s1, e->stream));
    // The GPU works for milliseconds from here: give the scheduler lock back so that submit / cancel / close /
    // drain / stats from other threads return at once (a submit used to wait for the whole step, which
    // serialised 64 sessions arriving together into 64 steps).  What they may do meanwhile is limited to state
    // this step does not use: requests in flight are only MARKED (cancel_pending / close_pending).
    for (Request* r : dec) r->in_flight = true;
    for (Request* r : pre) r->in_flight = true;
    lk.unlock();
    const cudaError_t sync_rc = cudaStreamSynchronize(e->stream);
    lk.lock();
    for (Request* r : dec) r->in_flight = false;
    for (Request* r : pre) r->in_flight = false;
    FT_CHECK_CUDA(sync_rc);
    e->st.d2h_bytes += (long long)b.n_logit_rows * sizeof(int);
    {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, e->s0, e->s1) == cudaSuccess) {
            if (e->step_log.size() >= kStepTimes) e->step_log.pop_front();
            const float host_ms =
                std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t_begin).count();
            e->step_log.push_back({ms, (float)b.n_decode, (float)(b.T - b.n_decode), host_ms});
        }
    }
    for (int l = 0; l < e->prof_used; ++l) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, e->prof_ev[2 * l], e->prof_ev[2 * l + 1]) == cudaSuccess) {
            e->st.attn_decode_ms += ms;
            e->st.attn_decode_launches++;
            e->st.attn_decode_kv_tokens += b.n_decode > 0 ? e->prof_ctx_sum : 0;
        }
    }

    // ---- bookkeeping: the K/V of every token we just ran is now cached
    int produced = 0;
    auto emit = [&](Request* r) {
        const int tok = h[m.o_sampled + r->logits_row];
        r->last_token = tok;
        r->n_generated++;
        produced++;
        bool is_eos = false;
        if (!r->ignore_eos)
            for (int k = 0; k < c.n_eos; ++k) is_eos |= tok == c.eos_ids[k];
        const int ctx_after = (int)r->sess->tokens.size() + 1;      // if this token were fed back
        if (is_eos) finish_request(e, r, 1, tok);
        else if (r->n_generated >= r->max_new || ctx_after >= c.max_context) finish_request(e, r, 2, tok);
        else e->out.push_back({r->id, tok, 0});
    };
    std::vector<Session*> to_close;
    auto settle = [&](Request* r) -> bool {      // true: the request was cancelled / its session closed mid-step
        if (r->sess && r->sess->close_pending && std::find(to_close.begin(), to_close.end(), r->sess) == to_close.end())
            to_close.push_back(r->sess);
        if (!r->cancel_pending) return false;
        r->cancel_pending = false;
        finish_request(e, r, 3, -1);
        return true;
    };
    for (Request* r : dec) {
        r->sess->tokens.push_back(r->last_token);
        if (!settle(r)) emit(r);
    }
    for (int j = 0; j < b.n_prefill_req; ++j) {
        Request* r = pre[j];
        Session* s = r->sess;
        s->tokens.insert(s->tokens.end(), r->prompt.begin() + r->prefill_pos,
                         r->prompt.begin() + r->prefill_pos + pre_len[j]);
        r->prefill_pos += pre_len[j];
        e->st.prefill_tokens += pre_len[j];
        if (settle(r)) continue;
        if (r->logits_row >= 0) {
            r->state = REQ_DECODE;
            emit(r);
        }
    }
    for (Session* sx : to_close) {
        for (auto& kv : e->requests)
            if (kv.second->sess == sx) kv.second->sess = nullptr;
        drop_session(e, sx);
    }
    e->st.steps++;
    if (b.n_decode > 0) e->st.decode_steps++;
    e->st.decode_tokens += b.n_decode;
    e->st.last_batch = b.n_req;
    e->st.last_prefill_tokens = b.T - b.n_decode;
    e->st.last_step_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_begin).count();
    return produced;
}

// The pinned + device block of per-step metadata (layout: StepMeta).
static int init_meta(Engine* e, size_t rows_last) {
    const ft_engine_config& c = e->cfg;
    const size_t T = e->t_max;
    StepMeta& m = e->meta;
    size_t o = 0;
    auto take = [&](size_t n) { size_t r = o; o += align4(n); return r; };
    const size_t R = e->r_max, LR = rows_last;
    const size_t max_tiles = T / 64 + R + 1;
    m.o_ctx = take(R); m.o_qstart = take(R + 1); m.o_rslot = take(R); m.o_rpos0 = take(R);
    m.o_treq = take(max_tiles); m.o_tq0 = take(max_tiles);
    m.o_lrow = take(LR); m.o_temp = take(LR); m.o_topk = take(LR); m.o_topp = take(LR);
    m.o_seed = take(2 * LR);
    m.o_xstart = take(R + 1); m.o_xpos0 = take(R); m.o_xslot = take(R);
    m.o_pt = take(0);
    o += align4(R * e->max_pages) + 3 * align4(T);      // page table + tokens | positions | rows
    m.o_tprefix = take(R + 1);
    m.o_sampled = take(LR);
    m.ints = o;
    layout_step(m, (int)R, e->max_pages, (int)T);
    FT_CHECK_CUDA(cudaMallocHost(&m.h, o * sizeof(int)));
    FT_CHECK_CUDA(cudaMalloc(&m.d, o * sizeof(int)));
    memset(m.h, 0, o * sizeof(int));
    FT_CHECK_CUDA(cudaMemsetAsync(m.d, 0, o * sizeof(int), e->stream));

    return 0;
}

static int init_events_and_pages(Engine* e) {
    const ft_engine_config& c = e->cfg;
    e->prof_ev.resize(2 * (size_t)std::max(e->cfg.layers, 1));
    for (auto& ev : e->prof_ev) FT_CHECK_CUDA(cudaEventCreate(&ev));
    FT_CHECK_CUDA(cudaEventCreate(&e->t0));
    FT_CHECK_CUDA(cudaEventCreate(&e->t1));
    FT_CHECK_CUDA(cudaEventCreate(&e->s0));
    FT_CHECK_CUDA(cudaEventCreate(&e->s1));
    e->free_pages.reserve(c.num_pages);
    for (int p = c.num_pages - 1; p >= 0; --p) e->free_pages.push_back(p);
    e->st.total_pages = c.num_pages;
    return 0;
}

static int engine_init_layered(Engine* e);

// ------------------------------------------------------------------ construction
static int engine_init(Engine* e) {
    if (e->lay) return engine_init_layered(e);
    const ft_engine_config& c = e->cfg;
    FT_REQUIRE(c.head_dim == 64 || c.head_dim == 128, "engine: head_dim %d not supported", c.head_dim);
    FT_REQUIRE(c.n_q_heads % c.n_kv_heads == 0 && c.n_q_heads / c.n_kv_heads <= 8,
               "engine: GQA group must divide and be <= 8");
    FT_REQUIRE(c.hidden % 128 == 0 && c.ffn % 64 == 0 && c.vocab % 128 == 0,
               "engine: hidden/vocab must be multiples of 128 and ffn of 64");
    FT_REQUIRE(c.max_batch >= 1 && c.max_batched_tokens >= c.max_batch, "engine: bad batch limits");
    FT_REQUIRE(c.max_context >= 64 && c.num_pages >= 1, "engine: bad context/page limits");
    FT_CHECK_CUDA(cudaGetDevice(&e->dev));
    FT_CHECK_CUDA(cudaDeviceGetAttribute(&e->sms, cudaDevAttrMultiProcessorCount, e->dev));
    int cc_major = 0;
    FT_CHECK_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, e->dev));
    FT_REQUIRE(cc_major == 10, "engine: needs an sm_100 GPU (found compute capability %d.x)", cc_major);
    FT_CHECK_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));

    e->q_dim = c.n_q_heads * c.head_dim;
    e->kv_dim = c.n_kv_heads * c.head_dim;
    e->qkv_dim = e->q_dim + 2 * e->kv_dim;
    FT_REQUIRE(e->qkv_dim % 128 == 0 && e->q_dim % 64 == 0, "engine: projection dims must tile");
    e->group = c.n_q_heads / c.n_kv_heads;
    e->max_pages = ceil_div(c.max_context, kKvTile);
    e->t_max = c.max_batched_tokens;
    e->r_max = c.max_batch;
    e->logit_rows = std::max(c.max_batch, c.debug_logit_rows);
    e->pdl = c.use_pdl != 0;
    e->prefill_planes = c.prefill_planes >= 1 && c.prefill_planes <= 3 ? c.prefill_planes : kDefaultPrefillPlanes;
    if (const char* ov = getenv("FT_PREFILL_PLANES"))       // A/B switch for experiments (scripts/)
        if (atoi(ov) >= 1 && atoi(ov) <= 3) e->prefill_planes = atoi(ov);
    e->decode_prefill_cap = c.decode_prefill_cap == 0 ? kDefaultDecodePrefillCap : c.decode_prefill_cap < 0 ? 0 : c.decode_prefill_cap;
    e->tp = c.tp_size > 1 ? c.tp_size : 1;
    FT_REQUIRE(e->tp <= 2 && c.tp_rank >= 0 && c.tp_rank < e->tp, "engine: tensor parallelism is built for 2 ranks");
    FT_REQUIRE(c.vocab % (128 * e->tp) == 0, "engine: vocab must split into 128-row tiles per rank");
    e->vocab_local = c.vocab / e->tp;
    e->kv_layer_bytes = (size_t)c.num_pages * c.n_kv_heads * 2 * kKvTile * c.head_dim * 2;

    const size_t T = e->t_max;
    FT_CHECK_CUDA(cudaMalloc(&e->kv, e->kv_layer_bytes * c.layers));
    FT_CHECK_CUDA(cudaMemsetAsync(e->kv, 0, e->kv_layer_bytes * c.layers, e->stream));
    FT_CHECK_CUDA(cudaMalloc(&e->resid, T * c.hidden * 4));
    const size_t rows_last = std::max<size_t>(e->logit_rows, 256);
    FT_CHECK_CUDA(cudaMalloc(&e->q, T * e->q_dim * 2));
    FT_CHECK_CUDA(cudaMalloc(&e->logits, (size_t)e->logit_rows * c.vocab * 4));
    if (e->tp > 1) {
        // plain cudaMalloc: these three are exported to the peer process through cudaIpc handles
        FT_CHECK_CUDA(cudaMalloc(&e->tp_xchg, 2 * T * c.hidden * 4));
        FT_CHECK_CUDA(cudaMalloc(&e->tp_flags, kTpFlags * sizeof(unsigned)));
        FT_CHECK_CUDA(cudaMemsetAsync(e->tp_flags, 0, kTpFlags * sizeof(unsigned), e->stream));
    }
    auto alloc_zero = [&](void** p, size_t bytes) -> int {
        FT_CHECK_CUDA(cudaMalloc(p, bytes));
        FT_CHECK_CUDA(cudaMemsetAsync(*p, 0, bytes, e->stream));
        return 0;
    };
    FT_TRY(alloc_zero(&e->xn, T * c.hidden * 2));
    FT_TRY(alloc_zero(&e->xn_lo, T * c.hidden * 2));
    FT_TRY(alloc_zero(&e->attn_out, T * e->q_dim * 2));
    FT_TRY(alloc_zero(&e->attn_out_lo, T * e->q_dim * 2));
    FT_TRY(alloc_zero(&e->act, T * c.ffn * 2));
    FT_TRY(alloc_zero(&e->act_lo, T * c.ffn * 2));
    FT_TRY(alloc_zero(&e->xn_last, rows_last * c.hidden * 2));
    FT_TRY(alloc_zero(&e->xn_last_lo, rows_last * c.hidden * 2));
    // per-row-tile sums of squares of the residual rows (RMSNorm statistics, see forward())
    e->ssq_parts = c.hidden / 128;
    e->rows_last = (int)rows_last;
    {
        void* p = nullptr;
        FT_TRY(alloc_zero(&p, (size_t)e->ssq_parts * T * 4));
        e->ssq = static_cast<float*>(p);
        FT_TRY(alloc_zero(&p, (size_t)e->ssq_parts * rows_last * 4));
        e->ssq_last = static_cast<float*>(p);
        // a split-K grid never exceeds one CTA per SM, each parking at most a 128 x 128 fp32 tile
        FT_TRY(alloc_zero(&p, (size_t)e->sms * 128 * 128 * 4));
        e->gemm_scratch = static_cast<float*>(p);
        FT_TRY(alloc_zero(&p, (size_t)2 * e->sms * 4));
        e->gemm_sync = static_cast<int*>(p);
    }

    // decode attention: persistent grid = SMs x resident CTAs
    {
        int per_sm = attn_decode_ctas_per_sm(c.head_dim);
        FT_REQUIRE(per_sm >= 1, "engine: decode attention kernel does not fit on an SM (%s)", last_error());
        e->attn_ctas = e->sms * per_sm;
    }
    FT_CHECK_CUDA(cudaMalloc(&e->attn_scratch,
                             attn_decode_scratch_floats(e->r_max, c.n_kv_heads, e->group, c.head_dim,
                                                        e->attn_ctas) * 4));

    FT_TRY(init_meta(e, rows_last));

    // tensor maps
    const size_t L = c.layers;
    e->m_wqkv.resize(L); e->m_wo.resize(L); e->m_wgu.resize(L); e->m_wd.resize(L);
    auto at = [](const void* p, size_t elems) { return (const void*)((const uint8_t*)p + elems * 2); };
    for (size_t l = 0; l < L; ++l) {
        FT_TRY(make_tmap_bf16_k64(&e->m_wqkv[l], at(e->w.wqkv, l * e->qkv_dim * c.hidden), e->qkv_dim, c.hidden, 128));
        FT_TRY(make_tmap_bf16_k64(&e->m_wo[l], at(e->w.wo, l * (size_t)c.hidden * e->q_dim), c.hidden, e->q_dim, 128));
        FT_TRY(make_tmap_bf16_k64(&e->m_wgu[l], at(e->w.wgu, l * 2 * (size_t)c.ffn * c.hidden), 2 * c.ffn, c.hidden, 128));
        FT_TRY(make_tmap_bf16_k64(&e->m_wd[l], at(e->w.wd, l * (size_t)c.hidden * c.ffn), c.hidden, c.ffn, 128));
    }
    FT_TRY(make_tmap_bf16_k64(&e->m_lm, e->w.lm_head, e->vocab_local, c.hidden, 128));
    for (int i = 0; i < 4; ++i) {
        // activation maps span the whole buffer; rows past the step's T hold stale (finite) data
        // whose output columns the GEMM epilogue masks
        FT_TRY(make_tmap_bf16_k64(&e->m_xn[i], e->xn, (int)T, c.hidden, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_xn_lo[i], e->xn_lo, (int)T, c.hidden, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_attn[i], e->attn_out, (int)T, e->q_dim, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_attn_lo[i], e->attn_out_lo, (int)T, e->q_dim, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_act[i], e->act, (int)T, c.ffn, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_act_lo[i], e->act_lo, (int)T, c.ffn, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_last[i], e->xn_last, (int)rows_last, c.hidden, kBns[i]));
        FT_TRY(make_tmap_bf16_k64(&e->m_last_lo[i], e->xn_last_lo, (int)rows_last, c.hidden, kBns[i]));
    }
    if (e->prefill_planes == 3) {
        // fp16 copies of the projection weights (bf16 -> fp16 is exact for every weight above fp16's subnormal range) and
        // fp16 staging planes of their inputs
        auto to16 = [&](void** dst, const void* src, size_t elems) -> int {
            FT_CHECK_CUDA(cudaMalloc(dst, elems * 2));
            return launch_planes_to_f16(src, nullptr, *dst, elems, false, e->stream);
        };
        FT_TRY(to16(&e->w16_qkv, e->w.wqkv, L * e->qkv_dim * c.hidden));
        FT_TRY(to16(&e->w16_o, e->w.wo, L * (size_t)c.hidden * e->q_dim));
        FT_TRY(to16(&e->w16_gu, e->w.wgu, L * 2 * (size_t)c.ffn * c.hidden));
        FT_TRY(to16(&e->w16_d, e->w.wd, L * (size_t)c.hidden * c.ffn));
        FT_TRY(alloc_zero(&e->x16_xn, T * c.hidden * 2));
        FT_TRY(alloc_zero(&e->x16_attn, T * e->q_dim * 2));
        FT_TRY(alloc_zero(&e->x16_act, T * c.ffn * 2));
        e->m16_wqkv.resize(L); e->m16_wo.resize(L); e->m16_wgu.resize(L); e->m16_wd.resize(L);
        for (size_t l = 0; l < L; ++l) {
            FT_TRY(make_tmap_bf16_k64(&e->m16_wqkv[l], at(e->w16_qkv, l * e->qkv_dim * c.hidden), e->qkv_dim, c.hidden, 128));
            FT_TRY(make_tmap_bf16_k64(&e->m16_wo[l], at(e->w16_o, l * (size_t)c.hidden * e->q_dim), c.hidden, e->q_dim, 128));
            FT_TRY(make_tmap_bf16_k64(&e->m16_wgu[l], at(e->w16_gu, l * 2 * (size_t)c.ffn * c.hidden), 2 * c.ffn, c.hidden, 128));
            FT_TRY(make_tmap_bf16_k64(&e->m16_wd[l], at(e->w16_d, l * (size_t)c.hidden * c.ffn), c.hidden, c.ffn, 128));
        }
        const int boxes[2] = {128, 64};
        for (int i = 0; i < 2; ++i) {         // 16-bit tiles: the tensor map only moves bits, the MMA descriptor names the type
            FT_TRY(make_tmap_bf16_k64(&e->m16_xn[i], e->x16_xn, (int)T, c.hidden, boxes[i]));
            FT_TRY(make_tmap_bf16_k64(&e->m16_attn[i], e->x16_attn, (int)T, e->q_dim, boxes[i]));
            FT_TRY(make_tmap_bf16_k64(&e->m16_act[i], e->x16_act, (int)T, c.ffn, boxes[i]));
        }
    }
    FT_TRY(init_events_and_pages(e));
    FT_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    return 0;
}

static int engine_init_layered(Engine* e) {
    const ft_engine_config& c = e->cfg;
    Layered& L = *e->lay;
    const ft_layered_model& M = L.m;
    FT_REQUIRE(M.width >= 1 && M.vocab >= 1 && M.n_layers >= 1, "engine: a layered model needs width, vocab and layers");
    FT_REQUIRE(c.max_batch >= 1 && c.max_batched_tokens >= c.max_batch, "engine: bad batch limits");
    FT_REQUIRE(c.max_context >= 1 && c.num_pages >= 1, "engine: bad context/page limits");
    FT_CHECK_CUDA(cudaGetDevice(&e->dev));
    FT_CHECK_CUDA(cudaDeviceGetAttribute(&e->sms, cudaDevAttrMultiProcessorCount, e->dev));
    int cc_major = 0;
    FT_CHECK_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, e->dev));
    FT_REQUIRE(cc_major == 10, "engine: needs an sm_100 GPU (found compute capability %d.x)", cc_major);
    FT_CHECK_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    e->max_pages = ceil_div(c.max_context, kKvTile);
    e->t_max = c.max_batched_tokens;
    e->r_max = c.max_batch;
    e->logit_rows = std::max(c.max_batch, c.debug_logit_rows);
    e->pdl = false;
    e->tp = 1;
    e->vocab_local = M.vocab;
    e->decode_prefill_cap = c.decode_prefill_cap == 0 ? kDefaultDecodePrefillCap : c.decode_prefill_cap < 0 ? 0 : c.decode_prefill_cap;

    // sizes over all layers; places of each layer in the latent cache and in a state slot
    size_t cache_floats = 0, buf = 1, act_cols = 1;
    size_t kv_floats = 0, br_q = 0, br_v = 0, br_o = 0, br_fin = 0, br_heads = 0, e_max_s = 1, scan_cn = 0;
    int n_in_max = 1, top_max = 1, heads_max = 1, rank_max = 0;
    size_t vfirst_cols = 0, lstage_cols = 0;
    bool use_hist = false;
    for (int l = 0; l < M.n_layers; ++l) {
        LayeredLayer& ll = L.layers[l];
        const ft_layer_desc& d = ll.d;
        FT_REQUIRE(d.n_in >= 1 && d.w_in, "engine: layer %d is incomplete", l);
        const bool hyper = d.form == FT_LAYER_HYPER;
        const bool sandwich = d.form == FT_LAYER_SANDWICH || hyper;      // forms whose feed-forward has projections of its own
        const bool post = d.form == FT_LAYER_POSTNORM;
        FT_REQUIRE(post == (L.layers[0].d.form == FT_LAYER_POSTNORM), "engine: post-norm layers do not mix with other layer forms");
        FT_REQUIRE(hyper == (L.layers[0].d.form == FT_LAYER_HYPER), "engine: hyper-connected layers do not mix with other layer forms");
        if (hyper) {
            FT_REQUIRE(d.norm_pre1 && (d.ff_kind == FT_FF_NONE || d.norm_pre2), "engine: hyper-connected layer %d lacks norm gains", l);
            FT_REQUIRE(M.streams <= 16 && M.final_norm_w, "engine: a hyper-connected model has 1 to 16 streams and a last norm with gains");
            FT_REQUIRE(d.mixer == FT_MIXER_BRANCHES || (d.mixer == FT_MIXER_CHANNEL_DELTA && d.rank_a == 0 && d.rank_g == 0),
                       "engine: hyper-connected layer %d takes branch mixers or the delta rule with one decay per head", l);
            L.hyper = true;
        } else if (post) {
            FT_REQUIRE(d.norm_post1 && (d.ff_kind == FT_FF_NONE || (d.ff_kind == FT_FF_DENSE && d.norm_post2)),
                       "engine: post-norm layer %d lacks norm gains (its feed-forward is dense or absent)", l);
            FT_REQUIRE(d.canon_taps >= 0 && d.canon_taps <= 17 && (d.canon_taps == 0 || (d.canon1 && (d.ff_kind == FT_FF_NONE || d.canon2))),
                       "engine: post-norm layer %d: bad input convolutions", l);
            L.postnorm = true;
            if (d.canon_taps > 1) {
                for (int k = 0; k < (d.ff_kind == FT_FF_NONE ? 1 : 2); ++k) {
                    ll.canon_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)(d.canon_taps - 1) * M.width;
                }
                L.slot_stride = (L.slot_stride + 3) & ~size_t(3);
                L.n_stateful++;
            }
            if (d.depth_w) use_hist = true;
        } else if (d.form == FT_LAYER_SANDWICH) {
            FT_REQUIRE(d.norm_pre1 && d.norm_post1 && (d.ff_kind == FT_FF_NONE || (d.norm_pre2 && d.norm_post2)),
                       "engine: sandwich layer %d lacks norm gains", l);
        } else {
            FT_REQUIRE(d.form == FT_LAYER_GATED && d.rg_bias && d.o_rg1 >= 0 && d.mixer != FT_MIXER_BRANCHES,
                       "engine: gated layer %d is incomplete (it takes latent attention or channel delta)", l);
        }
        n_in_max = std::max(n_in_max, d.n_in);
        if (d.mixer != FT_MIXER_BRANCHES) {
            FT_REQUIRE(d.heads >= 1 && d.dim >= 1 && d.vdim >= 1 && d.w_o, "engine: layer %d is incomplete", l);
            heads_max = std::max(heads_max, d.heads);
            buf = std::max(buf, (size_t)d.heads * d.vdim);
        }
        if (d.mixer == FT_MIXER_BRANCHES) {
            FT_REQUIRE(d.n_branches == 1 || d.n_branches == 2, "engine: layer %d has %d branches", l, d.n_branches);
            for (int k = 0; k < d.n_branches; ++k) {
                const ft_branch_desc& c = d.branch[k];
                FT_REQUIRE(c.heads >= 1 && c.kv_heads >= 1 && c.heads % c.kv_heads == 0 && c.dim >= 1 && c.vdim >= 1 && c.w_o &&
                               (c.kind == FT_BRANCH_SELECTIVE_SCAN || (c.o_q >= 0 && (c.o_k >= 0 || c.kv_lender > 0))),
                           "engine: layer %d branch %d is incomplete", l, k);
                const size_t hv = (size_t)c.heads * c.vdim;
                br_heads = std::max(br_heads, (size_t)c.heads);
                br_fin = std::max(br_fin, hv);
                if (c.kind == FT_BRANCH_WINDOW_ATTENTION) {
                    FT_REQUIRE(c.window >= 0 && (c.rot_dims == 0 || c.rot_freq), "engine: layer %d branch %d: bad window or rotation", l, k);
                    FT_REQUIRE(c.keep_first >= 0 && (!c.rel || c.rel_n >= 1) && (c.v_role == 0 || c.o_v >= 0) && (c.v_role != 2 || c.v_mix),
                               "engine: layer %d branch %d: incomplete attention options", l, k);
                    FT_REQUIRE(c.qk_norm >= 0 && c.qk_norm <= 2 && (!c.chunked || c.window > 0) && c.conv >= 0 && c.conv <= 16 &&
                                   (c.conv <= 1 || c.conv_w),
                               "engine: layer %d branch %d: bad norm, chunk or convolution options", l, k);
                    if (c.kv_lender > 0) {
                        // the keys and values of an earlier layer: same key heads and sizes, no cache of its own
                        FT_REQUIRE(c.kv_lender - 1 < l && c.v_role == 0, "engine: layer %d reads the keys of layer %d, which does not precede it", l,
                                   c.kv_lender - 1);
                        const ft_layer_desc& src = L.layers[c.kv_lender - 1].d;
                        int found = -1;
                        for (int j = 0; j < (src.mixer == FT_MIXER_BRANCHES ? src.n_branches : 0) && found < 0; ++j)
                            if (src.branch[j].kind == FT_BRANCH_WINDOW_ATTENTION && src.branch[j].kv_lender == 0) found = j;
                        FT_REQUIRE(found >= 0 && src.branch[found].kv_heads == c.kv_heads && src.branch[found].dim == c.dim &&
                                       src.branch[found].vdim == c.vdim && src.branch[found].o_v >= 0,
                                   "engine: layer %d: layer %d has no keys and values of its sizes to lend", l, c.kv_lender - 1);
                        ll.lender_branch[k] = found;
                    } else {
                        ll.br_cache_off[k] = kv_floats;
                        kv_floats += (size_t)e->cfg.num_pages * kKvTile * c.kv_heads * (c.dim + c.vdim);
                    }
                    if (c.conv >= 1) {           // the last conv - 1 projected q | k | v rows of the sequence
                        const size_t ch = (size_t)c.heads * c.dim + (c.kv_lender > 0 ? 0 : (size_t)c.kv_heads * (c.dim + c.vdim));
                        FT_REQUIRE(c.kv_lender > 0 ? true : (c.o_k == c.o_q + c.heads * c.dim && c.o_v == c.o_k + c.kv_heads * c.dim),
                                   "engine: layer %d branch %d: convolved q, k, v are adjacent columns", l, k);
                        ll.br_x_off[k] = L.slot_stride;
                        L.slot_stride += ch * (size_t)(c.conv - 1);
                        br_v = std::max(br_v, ch);
                        if (c.conv > 1) L.n_stateful++;
                    }
                    br_q = std::max(br_q, (size_t)c.heads * c.dim);
                    if (c.v_role) {
                        FT_REQUIRE(vfirst_cols == 0 || vfirst_cols == (size_t)c.kv_heads * c.vdim,
                                   "engine: layer %d: value mixing needs the value sizes of its first layer", l);
                        FT_REQUIRE(c.v_role == 1 || vfirst_cols, "engine: layer %d mixes values before any layer kept them", l);
                        vfirst_cols = (size_t)c.kv_heads * c.vdim;
                    }
                } else if (c.kind == FT_BRANCH_LATENT_WINDOW) {
                    FT_REQUIRE(c.window >= 0 && c.kv_rank >= 1 && c.q_rank >= 1 && c.rot_dims >= 0 && (c.rot_dims == 0 || c.rot_freq) &&
                                   c.w_uq && c.w_uk_t && c.w_uv && c.q_norm && c.kv_norm,
                               "engine: latent-window layer %d branch %d is incomplete", l, k);
                    const size_t kd = (size_t)c.rot_dims + c.kv_rank;
                    ll.br_cache_off[k] = kv_floats;
                    kv_floats += (size_t)e->cfg.num_pages * kKvTile * kd;
                    br_q = std::max(br_q, (size_t)c.heads * kd);
                    br_fin = std::max(br_fin, (size_t)c.heads * c.kv_rank);
                    lstage_cols = std::max(lstage_cols, (size_t)c.heads * kd + kd);
                    buf = std::max(buf, std::max((size_t)c.q_rank, (size_t)c.heads * (c.dim + c.rot_dims)));
                } else if (c.kind == FT_BRANCH_DECAY_ATTENTION) {
                    FT_REQUIRE(c.kv_heads == c.heads && c.decay && c.out_norm && c.o_v >= 0 && c.o_g >= 0 &&
                                   c.o_k == c.o_q + c.heads * c.dim && c.o_v == c.o_k + c.heads * c.dim,
                               "engine: decay-attention layer %d branch %d is incomplete", l, k);
                    ll.br_s_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads * c.dim * c.vdim;
                    br_o = std::max(br_o, hv);
                    L.n_stateful++;
                } else if (c.kind == FT_BRANCH_MATRIX_MEMORY) {
                    FT_REQUIRE(c.kv_heads == c.heads && c.gate_bias && c.gate_cap > 0.f && c.out_norm && c.o_v >= 0 && c.o_g >= 0 &&
                                   c.o_i >= 0 && c.o_f >= 0,
                               "engine: matrix-memory layer %d branch %d is incomplete", l, k);
                    ll.br_s_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads * c.dim * (c.vdim + 1);
                    ll.br_x_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads;
                    br_v = std::max(br_v, (size_t)c.heads * (c.vdim + 1));
                    br_o = std::max(br_o, (size_t)c.heads * (c.vdim + 1));
                    L.n_stateful++;
                } else if (c.kind == FT_BRANCH_STATE_SPACE) {
                    const size_t ch = hv + (size_t)2 * c.kv_heads * c.dim;
                    FT_REQUIRE(c.conv >= 1 && c.conv_w && c.dt_bias && c.a_log && c.out_norm && c.norm_groups >= 1 &&
                                   c.o_v >= 0 && c.o_z >= 0 && c.o_dt >= 0 && c.o_k == c.o_v + (int)hv &&
                                   c.o_q == c.o_k + c.kv_heads * c.dim,
                               "engine: state-space layer %d branch %d is incomplete", l, k);
                    ll.br_s_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads * c.dim * c.vdim;
                    ll.br_x_off[k] = L.slot_stride;
                    L.slot_stride += ch * (size_t)std::max(c.conv - 1, 0);
                    br_v = std::max(br_v, ch);
                    br_o = std::max(br_o, hv);
                    L.n_stateful++;
                } else if (c.kind == FT_BRANCH_SELECTIVE_SCAN) {
                    FT_REQUIRE(c.vdim == 1 && c.conv >= 1 && c.conv <= 16 && c.conv_w && c.dt_bias && c.a_log && c.skip && c.dt_rank >= 1 &&
                                   c.w_x && c.w_dt && c.o_v >= 0 && c.o_z >= 0 && c.dim <= 256,
                               "engine: selective-scan layer %d branch %d is incomplete", l, k);
                    ll.br_s_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads * c.dim;
                    ll.br_x_off[k] = L.slot_stride;
                    L.slot_stride += (size_t)c.heads * (size_t)(c.conv - 1);
                    br_v = std::max(br_v, (size_t)c.heads);
                    scan_cn = std::max(scan_cn, (size_t)c.heads * (size_t)(c.dim + 1));
                    FT_REQUIRE(c.x_rows == 0 || c.x_rows >= c.dt_rank + 2 * c.dim, "engine: layer %d branch %d: x_rows below the low-rank row", l, k);
                    buf = std::max(buf, std::max((size_t)c.heads, (size_t)std::max(c.x_rows, c.dt_rank + 2 * c.dim)));
                    L.n_stateful++;
                } else {
                    FT_REQUIRE(false, "engine: layer %d branch %d has an unknown kind %d", l, k, c.kind);
                }
                L.slot_stride = (L.slot_stride + 3) & ~size_t(3);
            }
        } else if (d.mixer == FT_MIXER_LATENT_ATTENTION) {
            FT_REQUIRE(d.kv_rank >= 1 && d.w_uk_t && d.w_uv && d.dkv_norm && d.o_q >= 0 && d.o_dkv >= 0 && d.o_gate >= 0,
                       "engine: latent-attention layer %d is incomplete", l);
            ll.cache_off = cache_floats;
            cache_floats += (size_t)c.num_pages * kKvTile * d.kv_rank;
            buf = std::max(buf, (size_t)d.heads * d.kv_rank);
            rank_max = std::max(rank_max, d.kv_rank);
        } else if (d.mixer == FT_MIXER_CHANNEL_DELTA) {
            FT_REQUIRE(d.kv_heads >= 1 && d.heads % d.kv_heads == 0 && d.conv >= 1 && d.rank_a >= 0 && d.rank_g >= 0 &&
                           d.conv_w && (d.rank_a == 0 || d.w_a2) && (d.rank_g == 0 || d.w_g2) && d.dt_bias && d.a_log && d.out_norm &&
                           d.o_q >= 0 && d.o_beta >= 0 && d.o_a1 >= 0 && d.o_g1 >= 0,
                       "engine: channel-delta layer %d is incomplete", l);
            const size_t ch = (size_t)2 * d.kv_heads * d.dim + (size_t)d.heads * d.vdim;
            ll.s_off = L.slot_stride;
            L.slot_stride += (size_t)d.heads * d.dim * d.vdim;
            ll.tail_off = L.slot_stride;
            L.slot_stride += ch * (size_t)std::max(d.conv - 1, 0);
            L.slot_stride = (L.slot_stride + 3) & ~size_t(3);
            L.n_stateful++;
            buf = std::max(buf, std::max(ch, (size_t)d.heads * d.dim));
        } else {
            FT_REQUIRE(false, "engine: layer %d has an unknown mixer %d", l, d.mixer);
        }
        if (d.ff_kind == FT_FF_MOE) {
            FT_REQUIRE(d.experts >= 1 && d.top >= 1 && d.top <= d.experts && d.ff >= 1 && d.w_gu && d.w_down &&
                           (sandwich ? d.w_router != nullptr : d.o_router >= 0 && d.o_rg2 >= 0),
                       "engine: mixture-of-experts layer %d is incomplete", l);
            FT_REQUIRE(!sandwich || d.shared_ff == 0 || (d.w_shared_up && d.w_shared_down),
                       "engine: layer %d lacks the shared expert's weights", l);
            top_max = std::max(top_max, d.top);
            act_cols = std::max(act_cols, (size_t)std::max(d.ff, sandwich ? d.shared_ff : 0));
            FT_REQUIRE(d.router_rows == 0 || d.router_rows >= d.experts, "engine: layer %d: router_rows below the expert count", l);
            e_max_s = std::max(e_max_s, (size_t)std::max(d.experts, d.router_rows));
        } else if (d.ff_kind == FT_FF_DENSE) {
            FT_REQUIRE((sandwich || post) && d.ff >= 1 && d.w_gu && d.w_down, "engine: dense feed-forward layer %d is incomplete", l);
            act_cols = std::max(act_cols, (size_t)d.ff);
        } else {
            FT_REQUIRE(d.ff_kind == FT_FF_NONE, "engine: layer %d has an unknown feed-forward %d", l, d.ff_kind);
        }
    }
    L.ld_proj = (n_in_max + 3) & ~3;
    L.tensor = M.exact_f32 == 0;
    L.top_max = top_max;
    const size_t T = e->t_max, W = M.width;
    const size_t rows_last_min = std::max<size_t>(e->logit_rows, 256);
    auto alloc = [&](void* pp, size_t bytes) -> int {
        void** p = reinterpret_cast<void**>(pp);
        FT_CHECK_CUDA(cudaMalloc(p, std::max<size_t>(bytes, 16)));
        FT_CHECK_CUDA(cudaMemsetAsync(*p, 0, std::max<size_t>(bytes, 16), e->stream));
        return 0;
    };
    FT_TRY(alloc(&L.lat_cache, cache_floats * 4));
    if (M.exact_f32 == 0) FT_TRY(alloc(&L.lat_cache16, cache_floats * 2));
    FT_TRY(alloc(&L.state, L.slot_stride * (size_t)c.max_sessions * 4));
    if (kv_floats) FT_TRY(alloc(&L.kv_cache, kv_floats * 4));
    if (br_fin) {
        FT_TRY(alloc(&L.bq, T * br_q * 4));
        FT_TRY(alloc(&L.bv, T * br_v * 4));
        FT_TRY(alloc(&L.bo, T * br_o * 4));
        FT_TRY(alloc(&L.bfin, T * br_fin * 4));
        FT_TRY(alloc(&L.ab, T * br_heads * 2 * 4));
        FT_TRY(alloc(&L.gates, T * br_heads * 2 * 4));
        FT_TRY(alloc(&L.floor, T * br_heads * 4));
        FT_TRY(alloc(&L.mix2, T * W * 4));
        buf = std::max(buf, br_fin);               // the planes of an output projection's input
    }
    if (use_hist) FT_TRY(alloc(&L.hist, (size_t)(M.n_layers + 1) * T * W * 4));
    if (vfirst_cols) FT_TRY(alloc(&L.v_first, T * vfirst_cols * 4));
    if (lstage_cols) FT_TRY(alloc(&L.lstage, T * lstage_cols * 4));
    if (L.postnorm) FT_TRY(alloc(&L.resid2, T * W * 4));
    if (L.hyper) FT_TRY(alloc(&L.streams, T * (size_t)std::max(M.streams, 1) * W * 4));
    FT_TRY(alloc(&L.ffa, T * act_cols * 2 * 4));
    FT_TRY(alloc(&L.ffb, T * act_cols * 4));
    FT_TRY(alloc(&L.rlog, T * e_max_s * 4));
    FT_TRY(alloc(&e->resid, T * W * 4));
    FT_TRY(alloc(&L.hn, T * W * 4));
    FT_TRY(alloc(&L.proj, T * L.ld_proj * 4));
    if (L.tensor) {
        const size_t k_max = std::max(buf, W);
        FT_TRY(alloc(&L.pl_hi, std::max<size_t>(T, rows_last_min) * k_max * 2));
        FT_TRY(alloc(&L.pl_lo, std::max<size_t>(T, rows_last_min) * k_max * 2));
        FT_TRY(alloc(&L.hn_hi, T * W * 2));
        FT_TRY(alloc(&L.hn_lo, T * W * 2));
        FT_TRY(alloc(&L.mx_hi, T * top_max * W * 2));
        FT_TRY(alloc(&L.mx_lo, T * top_max * W * 2));
        FT_TRY(alloc(&L.ax_hi, T * top_max * act_cols * 2));
        FT_TRY(alloc(&L.ax_lo, T * top_max * act_cols * 2));
        FT_TRY(alloc(&L.gu, T * top_max * act_cols * 2 * 4));
    }
    FT_TRY(alloc(&L.b1, T * buf * 4));
    FT_TRY(alloc(&L.b2, T * buf * 4));
    if (scan_cn > 0) {                  // what the segments of a long request leave behind for one another
        L.scan_ws_rows = selective_scan_ws_rows((int)T);
        FT_TRY(alloc(&L.scan_ws, (size_t)L.scan_ws_rows * scan_cn * 4));
    }
    FT_TRY(alloc(&L.b3, T * buf * 4));
    FT_TRY(alloc(&L.b4, T * buf * 4));
    FT_TRY(alloc(&L.beta, T * heads_max * 4));
    if (rank_max > 0) FT_TRY(alloc(&L.attn_part, (size_t)kLatentSplitPairs * kLatentMaxSplits * (rank_max + 2) * 4));
    FT_TRY(alloc(&L.mix, T * W * 4));
    FT_TRY(alloc(&L.act, T * top_max * act_cols * 4));
    FT_TRY(alloc(&L.eout, T * top_max * W * 4));
    FT_TRY(alloc(&L.wts, T * top_max * 4));
    FT_TRY(alloc(&L.ids, T * top_max * 4));
    FT_TRY(alloc(&L.slot_token, T * top_max * 4));
    FT_TRY(alloc(&L.slot_pos, T * top_max * 4));
    {
        int e_max = 1;
        for (const LayeredLayer& ll : L.layers) e_max = std::max(e_max, ll.d.experts);
        FT_TRY(alloc(&L.seg, (size_t)(e_max + 1) * 4));
        FT_CHECK_CUDA(cudaMallocHost(&L.h_seg, (size_t)(e_max + 1) * 4));
        if (L.tensor) {
            for (int k = 0; k < Layered::kSide; ++k) {
                FT_CHECK_CUDA(cudaStreamCreateWithFlags(&L.side[k], cudaStreamNonBlocking));
                FT_CHECK_CUDA(cudaEventCreateWithFlags(&L.side_done[k], cudaEventDisableTiming));
            }
            FT_CHECK_CUDA(cudaEventCreateWithFlags(&L.main_ready, cudaEventDisableTiming));
        }
    }
    const size_t rows_last = std::max<size_t>(e->logit_rows, 256);
    e->rows_last = (int)rows_last;
    FT_TRY(alloc(&L.xlast, rows_last * W * 4));
    FT_TRY(alloc(&e->logits, (size_t)e->logit_rows * M.vocab * 4));
    for (int sl = c.max_sessions - 1; sl >= 0; --sl) e->free_slots.push_back(sl);
    FT_TRY(init_meta(e, rows_last));
    FT_TRY(init_events_and_pages(e));
    FT_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    return 0;
}

static void engine_free(Engine* e) {
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (auto& kv : e->sessions) delete kv.second;
    for (auto& kv : e->requests) delete kv.second;
    cudaFree(e->kv); cudaFree(e->resid); cudaFree(e->ssq); cudaFree(e->ssq_last); cudaFree(e->gemm_scratch); cudaFree(e->gemm_sync); cudaFree(e->xn); cudaFree(e->q);
    cudaFree(e->attn_out); cudaFree(e->act); cudaFree(e->xn_last); cudaFree(e->logits);
    cudaFree(e->tp_xchg); cudaFree(e->tp_flags);
    cudaFree(e->xn_lo); cudaFree(e->attn_out_lo); cudaFree(e->act_lo); cudaFree(e->xn_last_lo);
    cudaFree(e->attn_scratch); cudaFree(e->meta.d);
    cudaFree(e->w16_qkv); cudaFree(e->w16_o); cudaFree(e->w16_gu); cudaFree(e->w16_d);
    cudaFree(e->x16_xn); cudaFree(e->x16_attn); cudaFree(e->x16_act);
    if (e->lay) {
        Layered& L = *e->lay;
        cudaFree(L.lat_cache); cudaFree(L.lat_cache16); cudaFree(L.state); cudaFree(L.hn); cudaFree(L.proj); cudaFree(L.b1); cudaFree(L.b2); cudaFree(L.scan_ws);
        cudaFree(L.b3); cudaFree(L.b4); cudaFree(L.beta); cudaFree(L.attn_part); cudaFree(L.mix); cudaFree(L.act); cudaFree(L.eout);
        cudaFree(L.kv_cache); cudaFree(L.bq); cudaFree(L.bv); cudaFree(L.bo); cudaFree(L.bfin); cudaFree(L.ab); cudaFree(L.gates);
        cudaFree(L.hist); cudaFree(L.v_first); cudaFree(L.lstage); cudaFree(L.resid2); cudaFree(L.streams);
        cudaFree(L.floor); cudaFree(L.mix2); cudaFree(L.ffa); cudaFree(L.ffb); cudaFree(L.rlog);
        cudaFree(L.wts); cudaFree(L.xlast); cudaFree(L.ids); cudaFree(L.seg); cudaFree(L.slot_token);
        cudaFree(L.slot_pos); cudaFree(L.trail); cudaFree(L.pl_hi); cudaFree(L.pl_lo); cudaFree(L.hn_hi); cudaFree(L.hn_lo);
        cudaFree(L.mx_hi); cudaFree(L.mx_lo); cudaFree(L.ax_hi); cudaFree(L.ax_lo); cudaFree(L.gu);
        if (L.h_seg) cudaFreeHost(L.h_seg);
        for (int k = 0; k < Layered::kSide; ++k) {
            if (L.side[k]) cudaStreamDestroy(L.side[k]);
            if (L.side_done[k]) cudaEventDestroy(L.side_done[k]);
        }
        if (L.main_ready) cudaEventDestroy(L.main_ready);
        delete e->lay;
    }
    if (e->meta.h) cudaFreeHost(e->meta.h);
    for (auto ev : e->prof_ev) if (ev) cudaEventDestroy(ev);
    if (e->t0) cudaEventDestroy(e->t0);
    if (e->t1) cudaEventDestroy(e->t1);
    if (e->s0) cudaEventDestroy(e->s0);
    if (e->s1) cudaEventDestroy(e->s1);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

}  // namespace ft

// ------------------------------------------------------------------ C ABI (engine level)
using namespace ft;

extern "C" ft_engine* ft_engine_create(const ft_engine_config* cfg, const ft_weights* w) {
    if (!cfg || !w) { set_last_error("ft_engine_create: null argument"); return nullptr; }
    Engine* e = new (std::nothrow) Engine();
    if (!e) { set_last_error("ft_engine_create: out of host memory"); return nullptr; }
    e->cfg = *cfg;
    e->w = *w;
    if (e->cfg.max_sessions < e->cfg.max_batch) e->cfg.max_sessions = e->cfg.max_batch * 4;
    if (engine_init(e) != 0) { engine_free(e); return nullptr; }
    return reinterpret_cast<ft_engine*>(e);
}

extern "C" ft_engine* ft_engine_create_layered(const ft_engine_config* cfg, const ft_layered_model* model) {
    if (!cfg || !model || !model->layers || model->n_layers < 1) {
        set_last_error("ft_engine_create_layered: null argument");
        return nullptr;
    }
    Engine* e = new (std::nothrow) Engine();
    if (!e) { set_last_error("ft_engine_create_layered: out of host memory"); return nullptr; }
    e->cfg = *cfg;
    e->w = ft_weights{};
    e->lay = new Layered();
    e->lay->m = *model;
    e->lay->layers.resize(model->n_layers);
    for (int l = 0; l < model->n_layers; ++l) e->lay->layers[l].d = model->layers[l];
    e->lay->m.layers = nullptr;
    e->cfg.hidden = model->width;
    e->cfg.vocab = model->vocab;
    e->cfg.layers = model->n_layers;
    if (e->cfg.max_sessions < e->cfg.max_batch) e->cfg.max_sessions = e->cfg.max_batch * 4;
    if (engine_init(e) != 0) { engine_free(e); return nullptr; }
    return reinterpret_cast<ft_engine*>(e);
}

static bool runnable(const Engine* e);

// A session for `key`, made if there is none: the stalest idle session gives way when the table (or, for models with
// recurrent layers, the state slots) is full.  Under e->mu.
static Session* session_for(Engine* e, unsigned long long key, const char* who) {
    auto it = e->sessions.find(key);
    if (it != e->sessions.end()) return it->second;
    const bool need_slot = e->lay && e->lay->n_stateful > 0;
    if ((int)e->sessions.size() >= e->cfg.max_sessions || (need_slot && e->free_slots.empty())) {
        Session* victim = nullptr;
        for (auto& kv : e->sessions)
            if (!kv.second->busy && (!victim || kv.second->last_used < victim->last_used)) victim = kv.second;
        if (!victim) {
            set_last_error("%s: all %d sessions are busy", who, e->cfg.max_sessions);
            return nullptr;
        }
        for (auto& kv : e->requests)
            if (kv.second->sess == victim) kv.second->sess = nullptr;
        drop_session(e, victim);
    }
    Session* s = new Session();
    s->key = key;
    if (need_slot) {
        s->slot = e->free_slots.back();
        e->free_slots.pop_back();
    }
    e->sessions[key] = s;
    return s;
}

extern "C" int ft_engine_feed(ft_engine* h, int n_entries, const unsigned long long* keys, const int* counts,
                              const int* tokens, int n_want, const int* want_rows, float* logits_out) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && n_entries >= 1 && keys && counts && tokens && n_want >= 0, "ft_engine_feed: bad arguments");
    FT_REQUIRE(n_want == 0 || (want_rows && logits_out), "ft_engine_feed: wanted rows without a place for them");
    FT_REQUIRE(n_entries <= e->r_max, "ft_engine_feed: %d entries exceed max_batch %d", n_entries, e->r_max);
    FT_REQUIRE(n_want <= e->logit_rows, "ft_engine_feed: %d wanted rows exceed debug_logit_rows %d", n_want, e->logit_rows);
    std::lock_guard<std::mutex> sk(e->step_mu);
    std::lock_guard<std::mutex> dk(g_device_step_mu[e->dev % kMaxDevices]);
    DeviceGuard dg(e->dev);
    std::unique_lock<std::mutex> lk(e->mu);
    FT_REQUIRE(!e->loop_on && runnable(e) == false, "ft_engine_feed: the engine has requests of its own in flight");
    int total = 0;
    for (int i = 0; i < n_entries; ++i) {
        FT_REQUIRE(counts[i] >= 1, "ft_engine_feed: entry %d is empty", i);
        for (int j = 0; j < i; ++j) FT_REQUIRE(keys[i] != keys[j], "ft_engine_feed: session %llu appears twice", keys[i]);
        total += counts[i];
    }
    FT_REQUIRE(total <= e->t_max, "ft_engine_feed: %d tokens exceed max_batched_tokens %d", total, e->t_max);
    for (int i = 0; i < total; ++i)
        FT_REQUIRE(tokens[i] >= 0 && tokens[i] < e->cfg.vocab, "ft_engine_feed: token %d out of range at %d", tokens[i], i);
    for (int i = 0; i < n_want; ++i)
        FT_REQUIRE(want_rows[i] >= 0 && want_rows[i] < total, "ft_engine_feed: wanted row %d out of range", want_rows[i]);
    // sessions and pages first (a session being made may evict an idle one, never one of this step)
    std::vector<Session*> sess(n_entries);
    for (int i = 0; i < n_entries; ++i) {
        Session* s = session_for(e, keys[i], "ft_engine_feed");
        if (!s) return -2;
        FT_REQUIRE(!s->busy, "ft_engine_feed: session %llu has a generation in flight", keys[i]);
        s->busy = true;                      // not a candidate for eviction while the step is put together
        s->last_used = ++e->clock;
        sess[i] = s;
    }
    int rc = 0;
    for (int i = 0; i < n_entries && !rc; ++i) {
        const int after = (int)sess[i]->tokens.size() + counts[i];
        if (after > e->cfg.max_context) { set_last_error("ft_engine_feed: session %llu would pass the %d-token context window", keys[i], e->cfg.max_context); rc = -2; }
        else if (!ensure_pages(e, sess[i], after)) { set_last_error("ft_engine_feed: out of cache pages"); rc = -3; }
    }
    // decode rows first, then prompt portions; `place` = first row of entry i in the batch
    std::vector<Portion> dec, pre;
    std::vector<int> place(n_entries, 0), first(n_entries, 0);
    if (!rc) {
        int off = 0;
        for (int i = 0; i < n_entries; ++i) { first[i] = off; off += counts[i]; }
        int row = 0;
        for (int i = 0; i < n_entries; ++i)
            if (counts[i] == 1 && !sess[i]->tokens.empty()) {
                dec.push_back({sess[i], tokens + first[i], 1, (int)sess[i]->tokens.size()});
                place[i] = row++;
            }
        for (int i = 0; i < n_entries; ++i)
            if (!(counts[i] == 1 && !sess[i]->tokens.empty())) {
                pre.push_back({sess[i], tokens + first[i], counts[i], (int)sess[i]->tokens.size()});
                place[i] = row;
                row += counts[i];
            }
        Batch b;
        fill_batch(e, dec, pre, b);
        StepMeta& m = e->meta;
        for (int i = 0; i < n_want; ++i) {
            int en = n_entries - 1;
            while (first[en] > want_rows[i]) --en;
            m.h[m.o_lrow + i] = place[en] + (want_rows[i] - first[en]);
        }
        b.n_logit_rows = n_want;
        b.logit_rows_identity = false;
        rc = upload_meta(e);
        if (!rc) rc = forward(e, b);
        if (!rc && n_want > 0 &&
            cudaMemcpyAsync(logits_out, e->logits, (size_t)n_want * e->cfg.vocab * 4, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess) {
            set_last_error("ft_engine_feed: logits copy failed");
            rc = -1;
        }
        if (!rc) {
            const cudaError_t se = cudaStreamSynchronize(e->stream);
            if (se != cudaSuccess) { set_last_error("ft_engine_feed: %s", cudaGetErrorString(se)); rc = -1; }
        }
        if (!rc) {
            for (int i = 0; i < n_entries; ++i)
                sess[i]->tokens.insert(sess[i]->tokens.end(), tokens + first[i], tokens + first[i] + counts[i]);
            e->st.steps++;
            e->st.prefill_tokens += total - (long long)dec.size();
            e->st.decode_tokens += (long long)dec.size();
            if (!dec.empty()) e->st.decode_steps++;
            e->st.last_batch = n_entries;
        }
    }
    for (int i = 0; i < n_entries; ++i) sess[i]->busy = false;
    return rc;
}

extern "C" int ft_engine_debug_trail(ft_engine* h, int on) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && e->lay, "ft_engine_debug_trail: not a layered engine");
    std::lock_guard<std::mutex> sk(e->step_mu);
    DeviceGuard dg(e->dev);
    Layered& L = *e->lay;
    if (on && !L.trail) FT_CHECK_CUDA(cudaMalloc(&L.trail, (size_t)L.m.n_layers * e->t_max * L.m.width * 4));
    L.trail_on = on != 0;
    return 0;
}

extern "C" int ft_engine_debug_read_trail(ft_engine* h, float* host_out, int rows) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && e->lay && host_out && rows >= 1 && rows <= e->t_max, "ft_engine_debug_read_trail: bad arguments");
    std::lock_guard<std::mutex> sk(e->step_mu);
    DeviceGuard dg(e->dev);
    Layered& L = *e->lay;
    FT_REQUIRE(L.trail, "ft_engine_debug_read_trail: the trail is off");
    const size_t W = L.m.width;
    for (int l = 0; l < L.m.n_layers; ++l)
        FT_CHECK_CUDA(cudaMemcpy(host_out + (size_t)l * rows * W, L.trail + (size_t)l * e->t_max * W, (size_t)rows * W * 4,
                                 cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" void ft_engine_destroy(ft_engine* h) {
    if (!h) return;
    Engine* e = reinterpret_cast<Engine*>(h);
    {   // a thread still blocked in ft_engine_wait (a daemon thread of the host at interpreter exit) leaves first; the
        // mark is set before the stepping thread stops, so that the waiter wakes to "destroyed" and not to "loop ended"
        std::lock_guard<std::mutex> lk(e->mu);
        e->closing = true;
        e->cv_out.notify_all();
    }
    ft_engine_stop(h);
    {
        std::unique_lock<std::mutex> lk(e->mu);
        e->cv_out.notify_all();
        e->cv_out.wait_for(lk, std::chrono::seconds(2), [&] { return e->waiters == 0; });
    }
    DeviceGuard dg(e->dev);
    engine_free(e);
}

extern "C" long long ft_engine_submit(ft_engine* h, unsigned long long key, const int* tokens, int n,
                                      float temperature, int top_k, float top_p, int max_new,
                                      unsigned long long seed, int ignore_eos) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && tokens && n >= 1, "ft_engine_submit: bad arguments");
    FT_REQUIRE(max_new >= 1, "ft_engine_submit: max_new_tokens must be >= 1");
    FT_REQUIRE(n + 1 <= e->cfg.max_context, "ft_engine_submit: prompt of %d tokens does not fit the %d-token context window", n, e->cfg.max_context);
    for (int i = 0; i < n; ++i)
        FT_REQUIRE(tokens[i] >= 0 && tokens[i] < e->cfg.vocab, "ft_engine_submit: token %d out of range at %d", tokens[i], i);
    std::lock_guard<std::mutex> lk(e->mu);
    Session* s = session_for(e, key, "ft_engine_submit");
    if (!s) return -2;
    FT_REQUIRE(!s->busy, "ft_engine_submit: session %llu already has a generation in flight", key);
    // longest common prefix with the cached conversation; at least one token must run
    int lcp = 0;
    const int lim = std::min((int)s->tokens.size(), n - 1);
    while (lcp < lim && s->tokens[lcp] == tokens[lcp]) ++lcp;
    // a recurrent state stands at the END of what it has seen: it can be continued, not rewound
    if (e->lay && e->lay->n_stateful > 0 && lcp != (int)s->tokens.size()) lcp = 0;
    release_pages_beyond(e, s, lcp);
    e->st.prefix_hit_tokens += lcp;
    s->busy = true;
    s->last_used = ++e->clock;
    Request* r = new Request();
    r->id = e->next_req++;
    r->sess = s;
    r->prompt.assign(tokens, tokens + n);
    r->prefill_pos = lcp;
    r->temperature = temperature;
    r->top_k = top_k;
    r->top_p = top_p;
    r->max_new = max_new;
    r->seed = seed;
    r->ignore_eos = ignore_eos;
    e->requests[r->id] = r;
    e->waiting.push_back(r);
    e->cv_work.notify_one();
    return r->id;
}

extern "C" int ft_engine_tp_export(ft_engine* h, void** xchg, void** flags, void** logits) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && xchg && flags && logits, "ft_engine_tp_export: bad arguments");
    FT_REQUIRE(e->tp > 1, "ft_engine_tp_export: the engine was created without tensor parallelism");
    DeviceGuard dg(e->dev);
    FT_CHECK_CUDA(cudaStreamSynchronize(e->stream));       // the arrival words are zeroed
    *xchg = e->tp_xchg;
    *flags = e->tp_flags;
    *logits = e->logits;
    return 0;
}

extern "C" int ft_engine_tp_attach(ft_engine* h, void* peer_xchg, void* peer_flags, void* peer_logits) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && peer_xchg && peer_flags && peer_logits, "ft_engine_tp_attach: bad arguments");
    FT_REQUIRE(e->tp > 1, "ft_engine_tp_attach: the engine was created without tensor parallelism");
    std::lock_guard<std::mutex> lk(e->mu);
    e->peer_xchg = static_cast<float*>(peer_xchg);
    e->peer_flags = static_cast<unsigned*>(peer_flags);
    e->peer_logits = static_cast<float*>(peer_logits);
    return 0;
}

extern "C" int ft_ipc_export(void* device_ptr, unsigned char handle_out[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
    FT_REQUIRE(device_ptr && handle_out, "ft_ipc_export: bad arguments");
    cudaIpcMemHandle_t hd;
    FT_CHECK_CUDA(cudaIpcGetMemHandle(&hd, device_ptr));
    memcpy(handle_out, &hd, 64);
    return 0;
}

extern "C" int ft_ipc_open(const unsigned char handle[64], void** device_ptr_out) {
    FT_REQUIRE(handle && device_ptr_out, "ft_ipc_open: bad arguments");
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, 64);
    FT_CHECK_CUDA(cudaIpcOpenMemHandle(device_ptr_out, hd, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

extern "C" int ft_ipc_close(void* device_ptr) {
    FT_REQUIRE(device_ptr, "ft_ipc_close: null pointer");
    FT_CHECK_CUDA(cudaIpcCloseMemHandle(device_ptr));
    return 0;
}

extern "C" int ft_engine_step(ft_engine* h) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_step: null engine");
    FT_REQUIRE(e->tp == 1 || e->peer_xchg, "ft_engine_step: tensor-parallel engine has no peer attached");
    std::lock_guard<std::mutex> sk(e->step_mu);
    std::lock_guard<std::mutex> dk(g_device_step_mu[e->dev % kMaxDevices]);
    DeviceGuard dg(e->dev);
    std::unique_lock<std::mutex> lk(e->mu);
    FT_REQUIRE(!e->loop_on, "ft_engine_step: the engine runs its own stepping thread (ft_engine_start); stop it first");
    return engine_step(e, lk);
}

// ---- the engine's own stepping thread
static bool runnable(const Engine* e) {           // under e->mu
    for (const Request* r : e->waiting)
        if (r->state != REQ_DONE) return true;
    for (const Request* r : e->active)
        if (r->state != REQ_DONE) return true;
    return false;
}

static void loop_main(Engine* e) {
    // a fresh thread's current device is 0: make the engine's GPU current for the thread's whole life, so that the
    // per-step DeviceGuard has nothing to restore (restoring "device 0" from a rank that lives on another GPU creates a
    // context there — 0.4 s the first time)
    cudaSetDevice(e->dev);
    for (;;) {
        {
            std::unique_lock<std::mutex> lk(e->mu);
            e->cv_work.wait_for(lk, std::chrono::milliseconds(20), [&] { return e->loop_stop || runnable(e); });
            if (e->loop_stop) break;
            if (!runnable(e)) continue;
        }
        int rc;
        bool stepped;
        {
            std::lock_guard<std::mutex> sk(e->step_mu);
            std::lock_guard<std::mutex> dk(g_device_step_mu[e->dev % kMaxDevices]);
            DeviceGuard dg(e->dev);
            std::unique_lock<std::mutex> lk(e->mu);
            const long long before = e->st.steps;
            rc = engine_step(e, lk);
            stepped = e->st.steps != before;
            if (rc < 0) {
                e->loop_error = rc;
                e->loop_error_msg = ft_last_error();
            }
        }
        e->cv_out.notify_all();
        if (rc < 0) break;
        if (!stepped) std::this_thread::sleep_for(std::chrono::microseconds(200));    // waiting on pages / admission
    }
    {
        std::lock_guard<std::mutex> lk(e->mu);
        e->loop_on = false;
    }
    e->cv_out.notify_all();
}

extern "C" int ft_engine_start(ft_engine* h) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_start: null engine");
    FT_REQUIRE(e->tp == 1, "ft_engine_start: tensor-parallel ranks are stepped in lock step by their host (tp.py)");
    {
        std::lock_guard<std::mutex> lk(e->mu);
        if (e->loop_on) return 0;
        FT_REQUIRE(e->loop_error == 0, "ft_engine_start: the stepping thread failed earlier: %s", e->loop_error_msg.c_str());
    }
    if (e->loop_thread.joinable()) e->loop_thread.join();       // a loop that ended by itself
    {
        std::lock_guard<std::mutex> lk(e->mu);
        e->loop_stop = false;
        e->loop_on = true;
    }
    e->loop_thread = std::thread(loop_main, e);
    return 0;
}

extern "C" int ft_engine_stop(ft_engine* h) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_stop: null engine");
    {
        std::lock_guard<std::mutex> lk(e->mu);
        e->loop_stop = true;
    }
    e->cv_work.notify_all();
    if (e->loop_thread.joinable()) e->loop_thread.join();
    return 0;
}

extern "C" int ft_engine_wait(ft_engine* h, int timeout_ms) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_wait: null engine");
    std::unique_lock<std::mutex> lk(e->mu);
    FT_REQUIRE(!e->closing, "ft_engine_wait: the engine is being destroyed");
    ++e->waiters;
    e->cv_out.wait_for(lk, std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms),
                       [&] { return !e->out.empty() || e->loop_error != 0 || !e->loop_on || e->closing; });
    --e->waiters;
    if (e->closing) {
        e->cv_out.notify_all();              // ft_engine_destroy waits for the last waiter to leave
        set_last_error("ft_engine_wait: the engine is being destroyed");
        return -1;
    }
    if (e->loop_error != 0 && e->out.empty()) {
        set_last_error("ft_engine_wait: the stepping thread stopped: %s", e->loop_error_msg.c_str());
        return -1;
    }
    return (int)e->out.size();
}

extern "C" int ft_engine_drain(ft_engine* h, long long* req_ids, int* tokens, int* finish, int cap) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && req_ids && tokens && finish, "ft_engine_drain: bad arguments");
    std::lock_guard<std::mutex> lk(e->mu);
    int n = 0;
    while (n < cap && !e->out.empty()) {
        const OutTok& o = e->out.front();
        req_ids[n] = o.req; tokens[n] = o.token; finish[n] = o.finish;
        if (o.finish) {                 // the request is over: forget it
            auto it = e->requests.find(o.req);
            if (it != e->requests.end() && it->second->state == REQ_DONE) {
                Request* r = it->second;
                e->active.erase(std::remove(e->active.begin(), e->active.end(), r), e->active.end());
                e->waiting.erase(std::remove(e->waiting.begin(), e->waiting.end(), r), e->waiting.end());
                delete r;
                e->requests.erase(it);
            }
        }
        e->out.pop_front();
        ++n;
    }
    return n;
}

extern "C" int ft_engine_cancel(ft_engine* h, long long req) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_cancel: null engine");
    std::lock_guard<std::mutex> lk(e->mu);
    auto it = e->requests.find(req);
    if (it == e->requests.end() || it->second->state == REQ_DONE) return 1;    // nothing to cancel
    if (it->second->in_flight) {         // inside the running step: finished as "cancelled" when it returns
        it->second->cancel_pending = true;
        return 0;
    }
    finish_request(e, it->second, 3, -1);
    e->cv_out.notify_all();
    return 0;
}

extern "C" int ft_engine_session_close(ft_engine* h, unsigned long long key) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_session_close: null engine");
    std::lock_guard<std::mutex> lk(e->mu);
    auto it = e->sessions.find(key);
    if (it == e->sessions.end()) return 1;
    Session* s = it->second;
    if (s->busy)
        for (auto& kv : e->requests)
            if (kv.second->sess == s && kv.second->state != REQ_DONE) {
                if (kv.second->in_flight) {      // its pages are being read and written right now: close after the step
                    kv.second->cancel_pending = true;
                    s->close_pending = true;
                    return 0;
                }
                finish_request(e, kv.second, 3, -1);
            }
    for (auto& kv : e->requests)
        if (kv.second->sess == s) kv.second->sess = nullptr;
    drop_session(e, s);
    return 0;
}

extern "C" int ft_engine_stats_get(ft_engine* h, ft_engine_stats* out) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && out, "ft_engine_stats_get: bad arguments");
    std::lock_guard<std::mutex> lk(e->mu);
    e->st.active_requests = 0;
    for (Request* r : e->active) e->st.active_requests += r->state != REQ_DONE;
    e->st.waiting_requests = (int)e->waiting.size();
    e->st.live_sessions = (int)e->sessions.size();
    e->st.free_pages = (int)e->free_pages.size();
    *out = e->st;
    return 0;
}

extern "C" int ft_engine_set_decode_prefill_cap(ft_engine* h, int cap) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_set_decode_prefill_cap: null engine");
    std::lock_guard<std::mutex> lk(e->mu);
    e->decode_prefill_cap = cap == 0 ? kDefaultDecodePrefillCap : cap < 0 ? 0 : cap;
    return 0;
}

extern "C" int ft_engine_set_profile(ft_engine* h, int on) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_set_profile: null engine");
    std::lock_guard<std::mutex> lk(e->mu);
    e->profile = on != 0;
    return 0;
}

extern "C" int ft_engine_timer(ft_engine* h, int stop, float* ms_out) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e, "ft_engine_timer: null engine");
    std::lock_guard<std::mutex> sk(e->step_mu);
    std::lock_guard<std::mutex> lk(e->mu);
    DeviceGuard dg(e->dev);
    if (!stop) {
        FT_CHECK_CUDA(cudaEventRecord(e->t0, e->stream));
        return 0;
    }
    FT_REQUIRE(ms_out, "ft_engine_timer: null output");
    FT_CHECK_CUDA(cudaEventRecord(e->t1, e->stream));
    FT_CHECK_CUDA(cudaEventSynchronize(e->t1));
    FT_CHECK_CUDA(cudaEventElapsedTime(ms_out, e->t0, e->t1));
    return 0;
}

extern "C" int ft_engine_step_log(ft_engine* h, float* out, int cap_rows) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && out && cap_rows >= 0, "ft_engine_step_log: bad arguments");
    std::lock_guard<std::mutex> lk(e->mu);
    while ((int)e->step_log.size() > cap_rows) e->step_log.pop_front();
    int n = 0;
    for (const auto& r : e->step_log) {
        out[4 * n + 0] = r.gpu_ms; out[4 * n + 1] = r.n_decode; out[4 * n + 2] = r.n_prefill; out[4 * n + 3] = r.host_ms;
        ++n;
    }
    e->step_log.clear();
    return n;
}

extern "C" int ft_engine_get_logits(ft_engine* h, long long req, float* host_out) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && host_out, "ft_engine_get_logits: bad arguments");
    std::lock_guard<std::mutex> sk(e->step_mu);       // the logits buffer belongs to the step while one runs
    std::lock_guard<std::mutex> lk(e->mu);
    DeviceGuard dg(e->dev);
    auto it = e->requests.find(req);
    FT_REQUIRE(it != e->requests.end() && it->second->logits_row >= 0,
               "ft_engine_get_logits: request %lld has no logits from the last step", req);
    FT_CHECK_CUDA(cudaMemcpy(host_out, e->logits + (size_t)it->second->logits_row * e->cfg.vocab,
                             (size_t)e->cfg.vocab * 4, cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" int ft_debug_prefill_logits(ft_engine* h, const int* tokens, int n, int chunk, float* host_out) {
    Engine* e = reinterpret_cast<Engine*>(h);
    FT_REQUIRE(e && tokens && host_out && n >= 1, "ft_debug_prefill_logits: bad arguments");
    std::lock_guard<std::mutex> sk(e->step_mu);
    std::lock_guard<std::mutex> dk(g_device_step_mu[e->dev % kMaxDevices]);
    std::lock_guard<std::mutex> lk(e->mu);
    DeviceGuard dg(e->dev);
    FT_REQUIRE(e->active.empty() && e->waiting.empty(), "ft_debug_prefill_logits: engine must be idle");
    FT_REQUIRE(chunk >= 1 && chunk <= e->logit_rows && chunk <= e->t_max,
               "ft_debug_prefill_logits: chunk %d exceeds debug_logit_rows %d / max_batched_tokens %d", chunk,
               e->logit_rows, e->t_max);
    FT_REQUIRE(n + 1 <= e->cfg.max_context, "ft_debug_prefill_logits: too long");
    Session tmp;
    if (e->lay && e->lay->n_stateful > 0) {
        FT_REQUIRE(!e->free_slots.empty(), "ft_debug_prefill_logits: no free state slot");
        tmp.slot = e->free_slots.back();
        e->free_slots.pop_back();
    }
    if (!ensure_pages(e, &tmp, n)) {
        if (tmp.slot >= 0) e->free_slots.push_back(tmp.slot);
        set_last_error("ft_debug_prefill_logits: out of KV pages");
        return -3;
    }
    StepMeta& m = e->meta;
    int rc = 0;
    for (int p0 = 0; p0 < n && rc == 0; p0 += chunk) {
        const int len = std::min(chunk, n - p0);
        Batch b;
        fill_batch(e, {}, {Portion{&tmp, tokens + p0, len, p0}}, b);
        for (int k = 0; k < len; ++k) m.h[m.o_lrow + k] = k;
        b.n_logit_rows = len;
        b.logit_rows_identity = true;
        rc = upload_meta(e);
        if (!rc) rc = forward(e, b);
        if (!rc && cudaMemcpyAsync(host_out + (size_t)p0 * e->cfg.vocab, e->logits, (size_t)len * e->cfg.vocab * 4,
                                   cudaMemcpyDeviceToHost, e->stream) != cudaSuccess) {
            set_last_error("ft_debug_prefill_logits: logits copy failed");
            rc = -1;
        }
        if (!rc && cudaStreamSynchronize(e->stream) != cudaSuccess) {
            set_last_error("ft_debug_prefill_logits: %s", cudaGetErrorString(cudaGetLastError()));
            rc = -1;
        }
    }
    release_pages_beyond(e, &tmp, 0);
    if (tmp.slot >= 0) e->free_slots.push_back(tmp.slot);
    return rc;
}
