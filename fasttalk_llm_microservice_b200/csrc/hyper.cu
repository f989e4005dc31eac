// Kernels of the hyper-connected layer form (FT_LAYER_HYPER) and of what its mixers and feed-forward add to the family.
// Everything here is fp32: the streams, their small mixing matrices, norms, step sizes, decays and the recurrent state.
//
//   joint            the ONE kernel between two GEMM chains of a layer, one CTA per row: the sublayer's result (up to two branch
//                    outputs, each optionally divided by its root mean square over the width and multiplied by a gain; or the
//                    experts' rows) joins all streams at once, X_t <- sum_s mix[s][t] X_s + out[t] y; then the row that the next
//                    sublayer (or the head) reads, u = sum_s in[s] X_s, passes its layer norm and is written with its bf16
//                    planes.  A step's first joint fills the streams from the embedding table instead
//   scaled rows      the rows a mixture of experts reads when a chosen score multiplies the expert's input
//   selective scan   S[c][n] <- exp(A[c][n] dt_c) S[c][n] + dt_c x_c B_n,  y_c = S[c] . C + D_c x_c, gated by silu(z): a few
//                    lanes share a channel and hold its states in registers; a request's tokens in order
#include "common.cuh"
#include "ft_internal.h"

#include <algorithm>
#include <cstdint>

namespace ft {
namespace {

__device__ __forceinline__ float silu_h(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_h(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ float cta_total(float v, float* red) {      // red: >= 33 floats of shared memory
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

constexpr int kMaxStreams = 16;

// V consecutive columns of a row at once: 16-byte loads and stores of fp32 (8-byte ones of bf16) when V == 4.
template <int V>
__device__ __forceinline__ void ld_cols(float (&d)[V], const float* p) {
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else {
        d[0] = *p;
    }
}
template <int V>
__device__ __forceinline__ void st_cols(float* p, const float (&d)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(d[0], d[1], d[2], d[3]);
    else *p = d[0];
}
template <int V>
__device__ __forceinline__ void ld_cols_bf16(float (&d)[V], const __nv_bfloat16* p) {
    if constexpr (V == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        d[0] = __low2float(a); d[1] = __high2float(a); d[2] = __low2float(b); d[3] = __high2float(b);
    } else {
        d[0] = __bfloat162float(*p);
    }
}
template <int V>
__device__ __forceinline__ void st_planes(__nv_bfloat16* hi, __nv_bfloat16* lo, const float (&d)[V]) {
    __nv_bfloat16 h[V], l[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        h[i] = __float2bfloat16_rn(d[i]);
        l[i] = __float2bfloat16_rn(d[i] - __bfloat162float(h[i]));
    }
    if constexpr (V == 4) {
        *reinterpret_cast<uint2*>(hi) = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(lo) = *reinterpret_cast<const uint2*>(l);
    } else {
        *hi = h[0];
        *lo = l[0];
    }
}

// MS: streams a thread keeps in registers (the arrays are indexed by unrolled loops); V: columns per thread and pass (4 when
// the width is a multiple of four and every row starts on 16 bytes)
template <int MS, int V>
__global__ void __launch_bounds__(256) hyper_joint_kernel(HyperArgs a) {
    __shared__ float red[33];
    __shared__ float smix[kMaxStreams * kMaxStreams], sout[kMaxStreams], sin_[kMaxStreams];
    extern __shared__ __align__(16) float row[];  // [W]: the row the next norm reads
    const int t = blockIdx.x, W = a.W, S = a.S;
    const int c_first = threadIdx.x * V, c_step = blockDim.x * V;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) smix[i] = a.mix ? a.mix[i] : (i / S == i % S ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        sout[i] = a.out ? a.out[i] : 1.f;
        sin_[i] = a.in_next ? a.in_next[i] : 1.f;
    }
    float r0 = 1.f, r1 = 1.f;
    if (a.g0 || a.g1) {                          // branch results that are normed over the width before they are summed
        float q0 = 0.f, q1 = 0.f;
        for (int c = c_first; c < W; c += c_step) {
            float v[V];
            if (a.g0) {
                ld_cols<V>(v, a.y0 + (size_t)t * W + c);
#pragma unroll
                for (int i = 0; i < V; ++i) q0 = fmaf(v[i], v[i], q0);
            }
            if (a.g1) {
                ld_cols<V>(v, a.y1 + (size_t)t * W + c);
#pragma unroll
                for (int i = 0; i < V; ++i) q1 = fmaf(v[i], v[i], q1);
            }
        }
        if (a.g0) r0 = 1.f / sqrtf(cta_total(q0, red) / (float)W + a.eps);
        if (a.g1) r1 = 1.f / sqrtf(cta_total(q1, red) / (float)W + a.eps);
    }
    __syncthreads();
    float* X = a.X + (size_t)t * S * W;
    float total = 0.f;
    if (a.tokens) {
        const __nv_bfloat16* er = (const __nv_bfloat16*)a.embed + (size_t)a.tokens[t] * W;
        for (int c = c_first; c < W; c += c_step) {
            float x[V], u[V], sm[V];
            ld_cols_bf16<V>(x, er + c);
#pragma unroll
            for (int i = 0; i < V; ++i) x[i] *= a.embed_scale;
            for (int s = 0; s < S; ++s) st_cols<V>(X + (size_t)s * W + c, x);
#pragma unroll
            for (int i = 0; i < V; ++i) {
                float ui = 0.f;
                for (int s = 0; s < S; ++s) ui = fmaf(sin_[s], x[i], ui);
                u[i] = ui;
                total += ui;
                sm[i] = x[i] * (float)S;
            }
            st_cols<V>(row + c, u);
            if (a.sum_out) st_cols<V>(a.sum_out + (size_t)t * W + c, sm);
        }
    } else {
        for (int c = c_first; c < W; c += c_step) {
            float y[V], g[V], v[V];
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = 0.f;
            if (a.y0) {
                ld_cols<V>(v, a.y0 + (size_t)t * W + c);
                if (a.g0) {
                    ld_cols<V>(g, a.g0 + c);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] = v[i] * r0 * g[i];
                }
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = a.s0 * v[i];
            }
            if (a.y1) {
                ld_cols<V>(v, a.y1 + (size_t)t * W + c);
                if (a.g1) {
                    ld_cols<V>(g, a.g1 + c);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] = v[i] * r1 * g[i];
                }
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = fmaf(a.s1, v[i], y[i]);
            }
            for (int k = 0; k < a.top; ++k) {
                ld_cols<V>(v, a.eout + (size_t)a.slot_pos[(size_t)t * a.top + k] * W + c);
                const float wk = a.wt ? a.wt[(size_t)t * a.top + k] : 1.f;
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = a.wt ? fmaf(wk, v[i], y[i]) : y[i] + v[i];
            }
            float xs[MS][V];
#pragma unroll
            for (int s = 0; s < MS; ++s) {
                if (s < S) {
                    ld_cols<V>(xs[s], X + (size_t)s * W + c);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) xs[s][i] = 0.f;
                }
            }
            float u[V], sum[V];
#pragma unroll
            for (int i = 0; i < V; ++i) u[i] = sum[i] = 0.f;
#pragma unroll
            for (int to = 0; to < MS; ++to) {
                if (to < S) {
                    float nv[V];
#pragma unroll
                    for (int i = 0; i < V; ++i) nv[i] = 0.f;
#pragma unroll
                    for (int s = 0; s < MS; ++s)
                        if (s < S) {
                            const float m = smix[s * S + to];
#pragma unroll
                            for (int i = 0; i < V; ++i) nv[i] = fmaf(m, xs[s][i], nv[i]);
                        }
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        nv[i] = fmaf(sout[to], y[i], nv[i]);
                        u[i] = fmaf(sin_[to], nv[i], u[i]);
                        sum[i] += nv[i];
                    }
                    st_cols<V>(X + (size_t)to * W + c, nv);
                }
            }
#pragma unroll
            for (int i = 0; i < V; ++i) total += u[i];
            st_cols<V>(row + c, u);
            if (a.sum_out) st_cols<V>(a.sum_out + (size_t)t * W + c, sum);
        }
    }
    if (!a.hn) return;
    const float mean = cta_total(total, red) / (float)W;
    float dev = 0.f;
    for (int c = c_first; c < W; c += c_step) {
        float u[V];
        ld_cols<V>(u, row + c);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float d = u[i] - mean;
            dev = fmaf(d, d, dev);
        }
    }
    const float rstd = 1.f / sqrtf(cta_total(dev, red) / (float)W + a.eps);
    __nv_bfloat16 *hi = (__nv_bfloat16*)a.hi, *lo = (__nv_bfloat16*)a.lo;
    for (int c = c_first; c < W; c += c_step) {
        float u[V], w[V], b[V];
        ld_cols<V>(u, row + c);
        ld_cols<V>(w, a.nw + c);
#pragma unroll
        for (int i = 0; i < V; ++i) b[i] = 0.f;
        if (a.nb) ld_cols<V>(b, a.nb + c);
#pragma unroll
        for (int i = 0; i < V; ++i) u[i] = (u[i] - mean) * rstd * w[i] + b[i];
        st_cols<V>(a.hn + (size_t)t * W + c, u);
        if (hi) st_planes<V>(hi + (size_t)t * W + c, lo + (size_t)t * W + c, u);
    }
}

__global__ void __launch_bounds__(256) scaled_rows_kernel(const float* __restrict__ src, const float* __restrict__ wt,
                                                          const int* __restrict__ slot_pos, int top, float* __restrict__ dst,
                                                          __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo, int W) {
    const int i = blockIdx.x;
    const float w = wt[i];
    const float* s = src + (size_t)(i / top) * W;
    const size_t o = (size_t)slot_pos[i] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = w * s[c];
        if (dst) dst[o + c] = v;
        if (hi) {
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            hi[o + c] = h;
            lo[o + c] = __float2bfloat16_rn(v - __bfloat162float(h));
        }
    }
}

// LPC lanes (a power of two, neighbours in a warp) share a channel; lane s of them holds states s, s + LPC, s + 2 LPC, ...
// (at most kScanKeep each), so a CTA of 128 threads owns 128 / LPC channels.  A request's tokens are cut into segments of
// seg_len (a multiple of the chunk), blockIdx.z names the segment, and the recurrence being linear in S lets the segments
// run side by side in two launches:
//   phase 0  segment 0 of every request runs from the slot's state (zero for a fresh sequence) and writes its outputs; a
//            request of one segment ends here (its state returns to the slot).  Every other segment but the last runs from
//            ZERO and writes nothing but what it leaves behind: L_p[c][n], its own contribution to the state at its end, and
//            d_p[c], the sum of its step sizes (the decay of a whole segment is exp(A[c][n] d_p[c])).  Segment 0 leaves the
//            true state at its end as L_0
//   phase 1  segment p >= 1 folds S = L_0, S <- exp(A d_q) S + L_q for q = 1 .. p-1, runs its tokens from there and writes
//            their outputs; the last one returns the state to the slot
// A step without a long request is phase 0 alone.  The workspace row of a full segment is (its first row) / seg_len, which no
// two full segments share.  Inside a segment the tokens come in chunks of kScanChunk: what a chunk brings — dt, x, z of the
// CTA's channels, B and C — is copied asynchronously into one of two shared-memory buffers while the chunk before it is
// computed.  Per chunk: the step sizes pass softplus in place (all threads), then the tokens in order (the state is the only
// dependence from token to token; a channel's partial read-outs meet by shuffles and land where its dt was), then skip, gate
// and the store, again by all threads with the channels along the lanes.  Decays are 2^(dt A log2(e)).
constexpr int kScanThreads = 128, kScanKeep = 8, kScanChunk = 16, kScanSeg = 128;
__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
// 2^x for x <= 0 in one instruction (results below the normal range become zero)
__device__ __forceinline__ float ex2_h(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// LPC and KEEP (lanes per channel, states a lane keeps) are fixed at compile time: the loops over a lane's states unroll
// without guards beyond n < N and the shared-memory reads of a token get constant offsets.
template <int PHASE, int LPC, int KEEP>
__global__ void __launch_bounds__(kScanThreads, 4) selective_scan_kernel(ScanArgs a, int seg_len) {
    constexpr int lpc = LPC;
    extern __shared__ __align__(16) float ssm[];
    const int r = blockIdx.y, seg = blockIdx.z + PHASE;
    const int start = a.req_start[r], n_req_tok = a.req_start[r + 1] - start;
    if (n_req_tok <= 0) return;
    const int n_seg = (n_req_tok + seg_len - 1) / seg_len;
    if (PHASE == 0 ? (seg > 0 && seg >= n_seg - 1) : seg >= n_seg) return;
    const bool emit = PHASE == 1 || seg == 0, last = seg == n_seg - 1;
    const int seg_start = start + seg * seg_len, n_tok = min(seg_len, n_req_tok - seg * seg_len);
    const int per = kScanThreads / lpc, N = a.N;
    const int c0 = blockIdx.x * per, ci = threadIdx.x / lpc, s = threadIdx.x % lpc;
    const int c = c0 + ci;
    const bool live = c < a.channels;
    const int cc = live ? c : a.channels - 1;
    const int n_ch = min(per, a.channels - c0);              // channels of this CTA that exist
    const int stage_f = kScanChunk * (3 * per + 2 * N);
    float* Sg = a.state + (size_t)a.req_slot[r] * a.slot_stride + a.s_off + (size_t)cc * N;
    float* Lw = a.ws + (size_t)a.ws_rows * a.channels * N;    // behind the L rows: the segments' summed step sizes
    float S[KEEP], A[KEEP];
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int n = s + lpc * i;
        A[i] = n < N ? -expf(a.a_log[(size_t)cc * N + n]) * 1.4426950408889634f : 0.f;
        S[i] = 0.f;
    }
    if (seg == 0) {
        if (a.req_pos0[r] != 0) {
#pragma unroll
            for (int i = 0; i < KEEP; ++i) {
                const int n = s + lpc * i;
                if (n < N) S[i] = Sg[n];
            }
        }
    } else if (PHASE == 1) {
        const size_t q0 = (size_t)(start / seg_len);         // segment 0's row; the later full segments follow it in order
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int n = s + lpc * i;
            if (n < N) S[i] = a.ws[(q0 * a.channels + cc) * N + n];
        }
        for (int p = 1; p < seg; ++p) {
            const size_t q = (size_t)((start + p * seg_len) / seg_len);
            const float d = Lw[q * a.channels + cc];
#pragma unroll
            for (int i = 0; i < KEEP; ++i) {
                const int n = s + lpc * i;
                if (n < N) S[i] = fmaf(ex2_h(d * A[i]), S[i], a.ws[(q * a.channels + cc) * N + n]);
            }
        }
    }
    auto stage = [&](int ch, float* buf) {
        const int t0 = seg_start + ch * kScanChunk, nt = min(kScanChunk, n_tok - ch * kScanChunk);
        float *sdt = buf, *sx = sdt + kScanChunk * per, *sz = sx + kScanChunk * per, *sB = sz + kScanChunk * per, *sC = sB + kScanChunk * N;
        for (int i = threadIdx.x; i < nt * n_ch; i += kScanThreads) {
            const int k = i / n_ch, j = i - k * n_ch;
            const size_t t = (size_t)(t0 + k);
            cp_async4(sdt + k * per + j, a.dt_raw + t * a.ldd + c0 + j);
            cp_async4(sx + k * per + j, a.x + t * a.ldx + c0 + j);
            if (emit) cp_async4(sz + k * per + j, a.z + t * a.ldz + c0 + j);
        }
        for (int i = threadIdx.x; i < nt * N; i += kScanThreads) {
            const int k = i / N, n = i - k * N;
            const size_t t = (size_t)(t0 + k);
            cp_async4(sB + k * N + n, a.B + t * a.ldbc + n);
            if (emit) cp_async4(sC + k * N + n, a.C + t * a.ldbc + n);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_chunks = (n_tok + kScanChunk - 1) / kScanChunk;
    float dsum = 0.f;
    stage(0, ssm);
    for (int ch = 0; ch < n_chunks; ++ch) {
        float* buf = ssm + (ch & 1) * stage_f;
        float *sdt = buf, *sx = sdt + kScanChunk * per, *sz = sx + kScanChunk * per, *sB = sz + kScanChunk * per, *sC = sB + kScanChunk * N;
        const int t0 = seg_start + ch * kScanChunk, nt = min(kScanChunk, n_tok - ch * kScanChunk);
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                                     // chunk ch has landed; nobody still reads the other buffer
        if (ch + 1 < n_chunks) stage(ch + 1, ssm + ((ch + 1) & 1) * stage_f);
        for (int i = threadIdx.x; i < nt * n_ch; i += kScanThreads) {
            const int k = i / n_ch, j = i - k * n_ch;
            sdt[k * per + j] = softplus_h(sdt[k * per + j] + a.dt_bias[c0 + j]);
        }
        __syncthreads();
        auto token = [&](int k) -> float {
            const float dt = sdt[k * per + ci], dx = dt * sx[k * per + ci];
            dsum += dt;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < KEEP; ++i) {
                // no branch (all lanes of the warp reach the shuffles below together): a lane's states beyond N have A = 0
                // and read B = C = 0, so they stay zero and add nothing
                const int n = s + lpc * i;
                const bool has = n < N;
                const float bn = has ? sB[k * N + (has ? n : 0)] : 0.f;
                S[i] = fmaf(ex2_h(dt * A[i]), S[i], dx * bn);
                if (emit) y = fmaf(S[i], has ? sC[k * N + (has ? n : 0)] : 0.f, y);
            }
            if (emit) {
#pragma unroll
                for (int off = 1; off < lpc; off <<= 1) y += __shfl_xor_sync(0xffffffffu, y, off);
            }
            return y;
        };
        if (nt == kScanChunk) {                              // a whole chunk: four tokens at a time with their read-outs in
#pragma unroll 1                                             // registers, so that their loads and shuffles overlap
            for (int k0 = 0; k0 < kScanChunk; k0 += 4) {
                float y[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) y[k] = token(k0 + k);
                if (emit && s == 0) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) sdt[(k0 + k) * per + ci] = y[k];
                }
            }
        } else {
            for (int k = 0; k < nt; ++k) {
                const float y = token(k);
                if (emit && s == 0) sdt[k * per + ci] = y;   // every lane of the channel has read dt before the shuffles end
            }
        }
        if (emit) {
            __syncthreads();
            for (int i = threadIdx.x; i < nt * n_ch; i += kScanThreads) {
                const int k = i / n_ch, j = i - k * n_ch;
                a.out[(size_t)(t0 + k) * a.channels + c0 + j] = fmaf(a.skip[c0 + j], sx[k * per + j], sdt[k * per + j]) * silu_h(sz[k * per + j]);
            }
        }
    }
    if (!live) return;
    if (last) {
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int n = s + lpc * i;
            if (n < N) Sg[n] = S[i];
        }
    } else if (PHASE == 0) {
        const size_t q = (size_t)(seg_start / seg_len);
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int n = s + lpc * i;
            if (n < N) a.ws[(q * a.channels + c) * N + n] = S[i];
        }
        if (s == 0) Lw[q * a.channels + c] = dsum;
    }
}

}  // namespace

int launch_hyper_joint(const HyperArgs& a, int T, cudaStream_t stream) {
    FT_REQUIRE(a.X && a.S >= 1 && a.S <= kMaxStreams && a.W >= 1, "hyper joint: 1 to %d streams (got %d)", kMaxStreams, a.S);
    FT_REQUIRE(a.tokens ? a.embed != nullptr : (a.y0 || a.y1 || a.top > 0), "hyper joint: nothing to join");
    FT_REQUIRE((!a.g0 || a.y0) && (!a.g1 || a.y1) && (a.top == 0 || (a.eout && a.slot_pos)) && (!a.hn || a.nw),
               "hyper joint: missing operands");
    const size_t smem = (size_t)a.W * 4;
    // four columns per thread when every row of every operand starts on 16 bytes (bf16 rows on 8): the width decides it for
    // buffers of the engine's own allocation, so a model always takes the same path
    auto al = [](const void* p, size_t n) { return ((uintptr_t)p & (n - 1)) == 0; };
    const bool v4 = a.W % 4 == 0 && al(a.X, 16) && al(a.y0, 16) && al(a.y1, 16) && al(a.g0, 16) && al(a.g1, 16) && al(a.eout, 16) &&
                    al(a.nw, 16) && al(a.nb, 16) && al(a.hn, 16) && al(a.sum_out, 16) && al(a.embed, 8) && al(a.hi, 8) && al(a.lo, 8);
    if (v4) {
        if (a.S <= 4) hyper_joint_kernel<4, 4><<<T, 256, smem, stream>>>(a);
        else if (a.S <= 8) hyper_joint_kernel<8, 4><<<T, 256, smem, stream>>>(a);
        else hyper_joint_kernel<kMaxStreams, 1><<<T, 256, smem, stream>>>(a);
    } else {
        if (a.S <= 4) hyper_joint_kernel<4, 1><<<T, 256, smem, stream>>>(a);
        else if (a.S <= 8) hyper_joint_kernel<8, 1><<<T, 256, smem, stream>>>(a);
        else hyper_joint_kernel<kMaxStreams, 1><<<T, 256, smem, stream>>>(a);
    }
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int launch_scaled_rows(const float* src, const float* wt, const int* slot_pos, int top, float* dst, void* hi, void* lo, int pairs,
                       int W, cudaStream_t stream) {
    FT_REQUIRE(src && wt && slot_pos && top >= 1 && (dst || (hi && lo)), "scaled rows: missing operands");
    if (pairs <= 0) return 0;
    scaled_rows_kernel<<<pairs, 256, 0, stream>>>(src, wt, slot_pos, top, dst, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, W);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int selective_scan_ws_rows(int rows) { return rows / kScanSeg + 1; }

int launch_selective_scan(const ScanArgs& a, int n_req, cudaStream_t stream) {
    FT_REQUIRE(a.channels >= 1 && a.N >= 1 && a.N <= 32 * kScanKeep, "selective scan: 1 to %d states per channel (got %d)",
               32 * kScanKeep, a.N);
    FT_REQUIRE(a.x && a.dt_raw && a.B && a.C && a.z && a.dt_bias && a.a_log && a.skip && a.out && a.state, "selective scan: missing operands");
    FT_REQUIRE(n_req >= 1 && a.rows >= n_req, "selective scan: %d rows for %d requests", a.rows, n_req);
    // the longest request has at most rows - (n_req - 1) tokens; segments only when the workspace holds their rows
    int n_seg = (a.rows - (n_req - 1) + kScanSeg - 1) / kScanSeg;
    if (!a.ws || a.ws_rows < selective_scan_ws_rows(a.rows)) n_seg = 1;
    const int seg_len = n_seg > 1 ? kScanSeg : a.rows + 1;
    // lanes per channel: about four states per lane; more lanes when the grid would leave SMs idle
    int lpc = 1;
    while (lpc < 32 && lpc * 4 < a.N) lpc <<= 1;
    while (lpc < 32 && (long long)n_req * n_seg * ((a.channels * lpc + kScanThreads - 1) / kScanThreads) < 148 && lpc < a.N) lpc <<= 1;
    while (lpc * kScanKeep < a.N) lpc <<= 1;
    const int per = kScanThreads / lpc;
    const size_t smem = (size_t)2 * kScanChunk * (3 * per + 2 * a.N) * 4;
    const unsigned cx = (a.channels + per - 1) / per;
    const int need = (a.N + lpc - 1) / lpc, keep = need <= 2 ? 2 : need <= 4 ? 4 : kScanKeep;
    const dim3 g0(cx, n_req, std::max(1, n_seg - 1)), g1(cx, n_req, std::max(1, n_seg - 1));
#define FT_SCAN_ONE(L, K)                                                                                             \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            FT_CHECK_CUDA(cudaFuncSetAttribute(selective_scan_kernel<0, L, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            FT_CHECK_CUDA(cudaFuncSetAttribute(selective_scan_kernel<1, L, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        }                                                                                                             \
        selective_scan_kernel<0, L, K><<<g0, kScanThreads, smem, stream>>>(a, seg_len);                               \
        if (n_seg > 1) selective_scan_kernel<1, L, K><<<g1, kScanThreads, smem, stream>>>(a, seg_len);                \
    } while (0)
#define FT_SCAN(L)                                \
    do {                                          \
        if (keep == 2) FT_SCAN_ONE(L, 2);         \
        else if (keep == 4) FT_SCAN_ONE(L, 4);    \
        else FT_SCAN_ONE(L, 8);                   \
    } while (0)
    switch (lpc) {
        case 1: FT_SCAN(1); break;
        case 2: FT_SCAN(2); break;
        case 4: FT_SCAN(4); break;
        case 8: FT_SCAN(8); break;
        case 16: FT_SCAN(16); break;
        default: FT_SCAN(32); break;
    }
#undef FT_SCAN
#undef FT_SCAN_ONE
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace ft
