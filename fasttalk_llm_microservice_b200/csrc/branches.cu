// Kernels of the branch mixers and of the sandwich layer form (ft_branch_desc, FT_LAYER_SANDWICH).  Everything here is
// fp32: positions and angles, scores and softmax, norms, gates, decays and the recurrent state; the projections that feed
// these kernels come from the linear / tensor-core GEMMs of the layered family.
//
//   sandwich norm        x += rms(y) * post_gain;  hn = rms(x) * next_gain   (y = scaled sum of up to two branch results, or
//                        the experts' weighted sum plus the shared expert): one kernel between any two GEMMs of a layer
//   window attention     biases + rotary pairs, rotated keys and values into the paged cache; one CTA per (token, head),
//                        its warps take key blocks of the window in turn (one key per lane for the scores, one value column
//                        per lane for the sum), online softmax, merged through shared memory; prompt portions on a tiled
//                        kernel.  Options, each off by default: queries and keys divided by their root mean square, a bias
//                        by distance, first positions that stay visible beyond the window, a sink in the softmax denominator,
//                        values mixed with those an earlier layer kept for the step, values that are columns of the keys
//   scalar-decay rule    S <- a_t S + b_t k_t v_t^T, o_t = S^T q_t for a request's tokens in order; one CTA per (request,
//                        head, block of value columns), LPC lanes share a column and hold a run of key channels of its
//                        state in registers.  Decay attention, the gated matrix memory and the state-space mixer all run
//                        on it; they differ in how a, b, q, k, v are prepared and in the read-out that follows
//   preparation          SiLU in place; gate pre-activations and the running-maximum scan of the matrix memory; short causal
//                        convolution over a step's rows and the slot's tail, step sizes and decays of the state space
//   read-out             normaliser, skip, gates and group-wise RMS norm, one CTA per (token, norm group)
#include "common.cuh"
#include "ft_internal.h"

#include <algorithm>

namespace ft {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ float cta_sum(float v, float* red) {      // red: >= 33 floats of shared memory
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

__device__ __forceinline__ void put_planes(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t i, float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
}

// ------------------------------------------------------------------ sandwich norm
__global__ void __launch_bounds__(256) sandwich_norm_kernel(SandwichArgs a) {
    __shared__ float red[33];
    extern __shared__ float row[];
    const int t = blockIdx.x, W = a.W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float y = 0.f;
        if (a.y0) y = a.s0 * a.y0[(size_t)t * W + c];
        if (a.y1) y = fmaf(a.s1, a.y1[(size_t)t * W + c], y);
        if (a.top > 0) {
            float f = 0.f;
            for (int k = 0; k < a.top; ++k)
                f = fmaf(a.wt[(size_t)t * a.top + k], a.eout[(size_t)a.slot_pos[(size_t)t * a.top + k] * W + c], f);
            y += f;
        }
        row[c] = y;
        ss += y * y;
    }
    ss = cta_sum(ss, red);
    const float r1 = 1.f / sqrtf(ss / (float)W + a.eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = a.x[(size_t)t * W + c] + row[c] * r1 * a.post_w[c];
        a.x[(size_t)t * W + c] = v;
        row[c] = v;
        s2 += v * v;
    }
    s2 = cta_sum(s2, red);
    const float r2 = 1.f / sqrtf(s2 / (float)W + a.eps);
    __nv_bfloat16 *hi = (__nv_bfloat16*)a.hi, *lo = (__nv_bfloat16*)a.lo;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = row[c] * r2 * a.next_w[c];
        a.hn[(size_t)t * W + c] = v;
        if (hi) put_planes(hi, lo, (size_t)t * W + c, v);
    }
}

int launch_sandwich_norm(const SandwichArgs& a, int T, cudaStream_t stream) {
    FT_REQUIRE(a.x && a.hn && a.post_w && a.next_w && (a.y0 || a.y1 || a.top > 0), "sandwich norm: missing operands");
    sandwich_norm_kernel<<<T, 256, (size_t)a.W * 4, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ elementwise preparation
// x[t][c0 .. c0 + n) <- silu(x) in place, rows of stride ld
__global__ void silu_cols_kernel(float* __restrict__ x, int ld, int c0, int n) {
    float* r = x + (size_t)blockIdx.x * ld + c0;
    for (int c = threadIdx.x; c < n; c += blockDim.x) r[c] = silu_f(r[c]);
}
int launch_silu_cols(float* x, int ld, int c0, int n, int T, cudaStream_t stream) {
    silu_cols_kernel<<<T, 256, 0, stream>>>(x, ld, c0, n);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}
// ab[t][h] = (decay[h], 1)
__global__ void const_decay_kernel(const float* __restrict__ decay, float* __restrict__ ab, int heads, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { ab[2 * (size_t)i] = decay[i % heads]; ab[2 * (size_t)i + 1] = 1.f; }
}
int launch_const_decay(const float* decay, float* ab, int heads, int T, cudaStream_t stream) {
    const int n = T * heads;
    const_decay_kernel<<<(n + 255) / 256, 256, 0, stream>>>(decay, ab, heads, n);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ window attention
// Token t: q = proj[o_q ..] + bias, rotated, -> q_out; k = proj[o_k ..] + bias: the rotated key and the value (the key before
// rotation, or proj[o_v ..]) -> the cache row of its position: [kv_heads * dim keys | kv_heads * vdim values].
// One coordinate of a query or key head after bias, norm factor, gain and rotation.  idx: its place in the projection's run of
// heads; c: its place inside the head; gi0: where the head's gains start in `gain` (the same for all heads, or per head).
struct RotSpec { const float* freq; int dims, half_layout; float mag; };
__device__ __forceinline__ float rotated(const float* __restrict__ src, const float* __restrict__ bias, const float* __restrict__ gain,
                                         int gi0, int idx, int c, const RotSpec& r, float pos, float sc) {
    float me = (src[idx] + (bias ? bias[idx] : 0.f)) * sc;
    if (gain) me *= gain[gi0 + c];
    if (c >= r.dims) return me;
    const int half = r.dims >> 1;
    // partner and turning direction: (2i, 2i+1) pairs, or (i, i + dims / 2)
    const bool second = r.half_layout ? c >= half : (c & 1);
    const int oc = r.half_layout ? (second ? c - half : c + half) : (second ? c - 1 : c + 1);
    const int other = idx + (oc - c);
    float ot = (src[other] + (bias ? bias[other] : 0.f)) * sc;
    if (gain) ot *= gain[gi0 + oc];
    float sn, cs;
    sincosf(pos * r.freq[r.half_layout ? (second ? c - half : c) : (c >> 1)], &sn, &cs);
    sn *= r.mag;
    cs *= r.mag;
    return second ? me * cs + ot * sn : me * cs - ot * sn;
}
__global__ void __launch_bounds__(128) window_write_kernel(WindowArgs a) {
    extern __shared__ float inv[];             // qk_norm: 1 / rms of every query head, then of every key head
    const int t = blockIdx.x;
    const float* pr = a.proj + (size_t)t * a.ldp;
    const int p = a.positions[t];
    const float pos = (float)p;
    const int nq = a.H * a.dim, nk = a.G * a.dim, nv = a.G * a.vdim;
    const int nkh = a.no_kv ? 0 : a.G;            // key heads this layer forms itself
    if (a.qk_norm == 2) {
        // one root mean square over all heads of q, one over all heads of k
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        if (wid < 2 && (wid == 0 || nkh > 0)) {
            const float* src = pr + (wid == 0 ? a.o_q : a.o_k);
            const float* bias = wid == 0 ? a.q_bias : a.k_bias;
            const int n = wid == 0 ? nq : nk;
            float ss = 0.f;
            for (int d = lane; d < n; d += 32) {
                const float v = src[d] + (bias ? bias[d] : 0.f);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float r = 1.f / sqrtf(ss / (float)n + a.eps);
            for (int hh = lane; hh < (wid == 0 ? a.H : a.G); hh += 32) inv[(wid == 0 ? 0 : a.H) + hh] = r;
        }
        __syncthreads();
    } else if (a.qk_norm) {
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
        for (int hh = wid; hh < a.H + nkh; hh += nw) {
            const bool isq = hh < a.H;
            const float* src = pr + (isq ? a.o_q + hh * a.dim : a.o_k + (hh - a.H) * a.dim);
            const float* bias = isq ? (a.q_bias ? a.q_bias + hh * a.dim : nullptr) : (a.k_bias ? a.k_bias + (hh - a.H) * a.dim : nullptr);
            float ss = 0.f;
            for (int d = lane; d < a.dim; d += 32) {
                const float v = src[d] + (bias ? bias[d] : 0.f);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) inv[hh] = 1.f / sqrtf(ss / (float)a.dim + a.eps);
        }
        __syncthreads();
    }
    const RotSpec rs = {a.rot_freq, a.rot_dims, a.rot_half, a.rot_mag};
    const bool wide = a.qk_norm == 2;             // gains per (head, coordinate) instead of per coordinate
    for (int i = threadIdx.x; i < nq; i += blockDim.x)
        a.q_out[(size_t)t * nq + i] = rotated(pr + a.o_q, a.q_bias, a.q_gain, wide ? i - i % a.dim : 0, i, i % a.dim, rs, pos,
                                              a.qk_norm ? inv[i / a.dim] : 1.f);
    if (a.no_kv) return;
    const int* pt = a.page_table + (size_t)a.seq_rows[t] * a.max_pages;
    const bool alias = a.v_in_key >= 0;                // the values are columns of the keys: the row holds the keys only
    float* row = a.cache + ((size_t)pt[p >> 6] * 64 + (p & 63)) * (size_t)(alias ? nk : nk + nv);
    for (int i = threadIdx.x; i < nk; i += blockDim.x)
        row[i] = rotated(pr + a.o_k, a.k_bias, a.k_gain, wide ? i - i % a.dim : 0, i, i % a.dim, rs, pos,
                         a.qk_norm ? inv[a.H + i / a.dim] : 1.f);
    const float lam = a.v_role == 2 ? a.v_mix[0] : 0.f;
    for (int i = threadIdx.x; i < (alias ? 0 : nv); i += blockDim.x) {
        float v = a.o_v >= 0 ? pr[a.o_v + i] + (a.v_bias ? a.v_bias[i] : 0.f) : pr[a.o_k + i] + (a.k_bias ? a.k_bias[i] : 0.f);
        if (a.v_role == 1) a.v_first[(size_t)t * nv + i] = v;
        else if (a.v_role == 2) v = (1.f - lam) * v + lam * a.v_first[(size_t)t * nv + i];
        row[nk + i] = v;
    }
}

// two fp32 numbers in one 64-bit register and the two-wide fp32 multiply-add of sm_100 (each half rounds as the scalar one)
typedef unsigned long long f32x2;      // two fp32 numbers in one 64-bit register
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// 16-byte asynchronous copy global -> shared of which only the first src_bytes (0 or 16) are read, the rest filled with zeros
__device__ __forceinline__ void cp_async16_zfill(float* dst_smem, const float* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes) : "memory");
}

constexpr int kWinWarps = 4;
template <int VPL, bool VEC>
__global__ void __launch_bounds__(kWinWarps * 32) window_attn_kernel(WindowArgs a) {
    extern __shared__ float sh[];
    float* sq = sh;                                    // [dim]
    float* sm = sq + ((a.dim + 3) & ~3);               // [warps] running maxima
    float* sl = sm + kWinWarps;                        // [warps] running sums
    float* sacc = sl + kWinWarps;                      // [warps][vdim]
    const int h = blockIdx.y, t = blockIdx.x;      // tokens along x: a step may hold more rows than y allows
    const int g = h / (a.H / a.G);
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.positions[t];
    const int lo = a.window > 0 ? (a.chunked ? p - p % a.window : max(0, p - a.window + 1)) : 0;
    const int nf = min(a.keep_first, lo);              // kept first positions that lie before the window
    const int n = nf + p - lo + 1;                     // key idx < nf: position idx; otherwise position lo + idx - nf
    const int* pt = a.page_table + (size_t)a.seq_rows[t] * a.max_pages;
    const bool alias = a.v_in_key >= 0;
    const size_t rowsz = (size_t)a.G * (alias ? a.dim : a.dim + a.vdim);
    const size_t v_at = alias ? (size_t)g * a.dim + a.v_in_key : (size_t)a.G * a.dim + (size_t)g * a.vdim;
    for (int c = threadIdx.x; c < a.dim; c += blockDim.x) sq[c] = a.q_out[((size_t)t * a.H + h) * a.dim + c];
    __syncthreads();
    float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
    for (int b0 = wid * 32; b0 < n; b0 += kWinWarps * 32) {
        const int idx = b0 + lane;
        const int j = idx < nf ? idx : lo + idx - nf;
        const bool valid = idx < n;
        const int jj = valid ? j : p;
        const long long base = ((long long)pt[jj >> 6] * 64 + (jj & 63)) * (long long)rowsz;
        const float* kr = a.cache + base + (size_t)g * a.dim;
        float s = 0.f;
        if (VEC) {
#pragma unroll 8
            for (int c = 0; c < a.dim; c += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kr + c);
                const float4 qv = *reinterpret_cast<const float4*>(sq + c);
                s = fmaf(qv.x, kv.x, s); s = fmaf(qv.y, kv.y, s); s = fmaf(qv.z, kv.z, s); s = fmaf(qv.w, kv.w, s);
            }
        } else {
            for (int c = 0; c < a.dim; ++c) s = fmaf(sq[c], kr[c], s);
        }
        s *= a.scale;
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        if (a.rel) s += a.rel[(size_t)min(p - jj, a.rel_n - 1) * a.H + h];
        if (!valid) s = -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);            // 0 on the first block (m = -inf)
        const float pj = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[i] *= corr;
        m = m_new;
        // all 32 keys of the block, four at a time so that their value loads are in flight together; a lane beyond the block's
        // end holds weight 0 and the (valid) row of position p
        for (int x0 = 0; x0 < 32; x0 += 4) {
            if (x0 >= n - b0) break;
            float px[4];
            const float* vr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                px[u] = __shfl_sync(0xffffffffu, pj, x0 + u);
                const long long bx = __shfl_sync(0xffffffffu, base, x0 + u);
                vr[u] = a.cache + bx + v_at;
            }
            float vv[4][VPL];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int i = 0; i < VPL; ++i) {
                    const int c = lane + 32 * i;
                    vv[u][i] = c < a.vdim ? vr[u][c] : 0.f;
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int i = 0; i < VPL; ++i) acc[i] = fmaf(px[u], vv[u][i], acc[i]);
        }
    }
    if (lane == 0) { sm[wid] = m; sl[wid] = l; }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;
        if (c < a.vdim) sacc[(size_t)wid * a.vdim + c] = acc[i];
    }
    __syncthreads();
    float mm = sm[0];
    for (int w = 1; w < kWinWarps; ++w) mm = fmaxf(mm, sm[w]);
    float den = 0.f;
    if (a.sink) {
        mm = fmaxf(mm, a.sink[h]);
        den = expf(a.sink[h] - mm);
    }
    for (int w = 0; w < kWinWarps; ++w) den += sl[w] * expf(sm[w] - mm);
    for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
        float num = 0.f;
        for (int w = 0; w < kWinWarps; ++w) num += sacc[(size_t)w * a.vdim + c] * expf(sm[w] - mm);
        a.out[((size_t)t * a.H + h) * a.vdim + c] = num / den;
    }
}

// Prompt portions: one CTA per (key head, run of QT consecutive tokens of one request), QT = 64 / (query heads per key head),
// so that up to 64 query rows — the tokens of the run times the query heads of the group — share every key and value row
// that is brought into shared memory.  Keys are taken 32 at a time from the first one the run's first token sees to the
// run's last position: S = Q K^T (each thread 2 rows x 4 keys, keys interleaved by 8 so that the 16-byte reads of a warp fall
// into different banks), cap, per-row window mask, online softmax (a row's 8 threads are neighbouring lanes), P to shared
// memory, O = O * corr + P V (each warp 8 rows, each lane 4 value columns per 128).  All of it in fp32.
constexpr int WT_ROWS = 64, WT_KEYS = 32, WT_THREADS = 256;
template <int VK>
__global__ void __launch_bounds__(WT_THREADS) window_tile_kernel(WindowArgs a, WindowTiles tm, int QT, int subs) {
    extern __shared__ __align__(16) float wsh[];
    const bool alias = a.v_in_key >= 0;       // the values are columns v_in_key.. of the key rows: no value tile of their own
    const int ldq = a.dim + 4, ldv = alias ? ldq : a.vdim, ldp = WT_KEYS + 1;
    const int kvf = WT_KEYS * ldq + (alias ? 0 : WT_KEYS * ldv);      // floats of one staged key (+ value) tile
    float* Qs = wsh;                          // [64][dim + 4]
    float* KV = Qs + WT_ROWS * ldq;           // two tiles of [32][dim + 4] keys (+ [32][vdim] values): one in use, one arriving
    float* Ps = KV + 2 * kvf;                 // [64][33]
    float* cr = Ps + WT_ROWS * ldp;           // [64] rescale of a row's sums in this tile; at the end the row's softmax sum
    const int tile = blockIdx.x / subs, sub = blockIdx.x % subs, g = blockIdx.y, tid = threadIdx.x;
    const int j = tm.tile_req[tile];
    const int q0 = tm.tile_q0[tile] + sub * QT;
    const int n_j = tm.req_q_start[j + 1] - tm.req_q_start[j];
    if (sub * QT >= 64 || q0 >= n_j) return;
    const int ntok = min(QT, min(n_j - q0, 64 - sub * QT));
    const int row_base = tm.req_q_start[j] + q0, p_first = tm.req_pos0[j] + q0;
    const int* pt = a.page_table + (size_t)tm.req_slot[j] * a.max_pages;
    const int grp = a.H / a.G, rows_used = ntok * grp;
    const size_t rowsz = (size_t)a.G * (alias ? a.dim : a.dim + a.vdim);
    const int d4n = a.dim >> 2, v4n = alias ? 0 : a.vdim >> 2;
    for (int i = tid; i < WT_ROWS * d4n; i += WT_THREADS) {
        const int r = i / d4n, d4 = i - r * d4n;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_used)
            v = *reinterpret_cast<const float4*>(a.q_out + ((size_t)(row_base + r / grp) * a.H + g * grp + r % grp) * a.dim + 4 * d4);
        *reinterpret_cast<float4*>(Qs + r * ldq + 4 * d4) = v;
    }
    const int lo = a.window > 0 ? (a.chunked ? p_first - p_first % a.window : max(0, p_first - a.window + 1)) : 0, hi = p_first + ntok - 1;
    const int ry = tid >> 3, cx = tid & 7;            // scores: rows 2 ry, 2 ry + 1; keys cx, cx + 8, cx + 16, cx + 24 of the tile
    const int oy = tid >> 5, ox = tid & 31;           // sums: rows 8 oy .. 8 oy + 7; columns 4 ox .. 4 ox + 3 (+ 128)
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int pr[2];
    bool rv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) { rv[i] = 2 * ry + i < rows_used; pr[i] = p_first + (2 * ry + i) / grp; }
    f32x2 acc[8][VK][2];                              // value columns (4 ox, + 1) and (+ 2, + 3) of 8 rows, per 128 columns
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int k = 0; k < VK; ++k)
#pragma unroll
            for (int c = 0; c < 2; ++c) acc[r][k][c] = 0ull;
    // The key tiles of this CTA in order: first those of the kept first positions that lie before the window (keys below nf),
    // then those of the window up to the run's last position.  Tile it + 1 is copied asynchronously while tile it is used.
    const int nf = min(a.keep_first, lo);
    const int n0 = (nf + WT_KEYS - 1) / WT_KEYS, nt = n0 + (hi - lo) / WT_KEYS + 1;
    auto stage = [&](int it, float* buf) {
        const bool seg = it >= n0;
        const int k0 = seg ? lo + (it - n0) * WT_KEYS : it * WT_KEYS, kend = seg ? hi + 1 : nf;
        for (int i = tid; i < WT_KEYS * d4n; i += WT_THREADS) {
            const int c = i / d4n, d4 = i - c * d4n, key = k0 + c;
            const bool ok = key < kend;             // rows beyond the end are filled with zeros (a copy of no source bytes)
            const float* src = ok ? a.cache + ((size_t)pt[key >> 6] * 64 + (key & 63)) * rowsz + (size_t)g * a.dim + 4 * d4 : a.cache;
            cp_async16_zfill(buf + c * ldq + 4 * d4, src, ok ? 16 : 0);
        }
        for (int i = tid; i < WT_KEYS * v4n; i += WT_THREADS) {
            const int c = i / v4n, d4 = i - c * v4n, key = k0 + c;
            const bool ok = key < kend;
            const float* src = ok ? a.cache + ((size_t)pt[key >> 6] * 64 + (key & 63)) * rowsz + (size_t)a.G * a.dim + (size_t)g * a.vdim + 4 * d4
                                  : a.cache;
            cp_async16_zfill(buf + WT_KEYS * ldq + c * ldv + 4 * d4, src, ok ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, KV);
    for (int it = 0; it < nt; ++it) {
        const bool seg = it >= n0;
        const int k0 = seg ? lo + (it - n0) * WT_KEYS : it * WT_KEYS, kend = seg ? hi + 1 : nf;
        const float* Ks = KV + (it & 1) * kvf;
        const float* Vs = alias ? Ks + a.v_in_key : Ks + WT_KEYS * ldq;
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                               // tile `it` has landed; the last tile's sums are done with the other buffer and Ps
        if (it + 1 < nt) stage(it + 1, KV + ((it + 1) & 1) * kvf);
        // a score is summed in two halves, even and odd channels side by side in one packed register: the 16-byte reads of
        // queries and keys are already pairs of neighbouring channels, so every multiply-add is two-wide without a move
        float sc[2][4];
        f32x2 sc2[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) sc2[i][c] = 0ull;
        for (int d4 = 0; d4 < d4n; ++d4) {
            const ulonglong2 q0v = *reinterpret_cast<const ulonglong2*>(Qs + (2 * ry) * ldq + 4 * d4);
            const ulonglong2 q1v = *reinterpret_cast<const ulonglong2*>(Qs + (2 * ry + 1) * ldq + 4 * d4);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const ulonglong2 kv = *reinterpret_cast<const ulonglong2*>(Ks + (cx + 8 * c) * ldq + 4 * d4);
                sc2[0][c] = fma2(q0v.x, kv.x, sc2[0][c]); sc2[0][c] = fma2(q0v.y, kv.y, sc2[0][c]);
                sc2[1][c] = fma2(q1v.x, kv.x, sc2[1][c]); sc2[1][c] = fma2(q1v.y, kv.y, sc2[1][c]);
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float ev, od;
                unpack2(sc2[i][c], ev, od);
                sc[i][c] = ev + od;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float tmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = k0 + cx + 8 * c;
                float v = sc[i][c] * a.scale;
                if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
                const bool vis = rv[i] && key < kend && key <= pr[i] &&
                                 (a.window <= 0 || (a.chunked ? key >= pr[i] - pr[i] % a.window : key > pr[i] - a.window) || key < a.keep_first);
                if (a.rel && vis) v += a.rel[(size_t)min(pr[i] - key, a.rel_n - 1) * a.H + g * grp + (2 * ry + i) % grp];
                sc[i][c] = vis ? v : -INFINITY;
                tmax = fmaxf(tmax, sc[i][c]);
            }
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            const float m_new = fmaxf(m[i], tmax);
            float corr = 1.f, psum = 0.f;
            if (m_new == -INFINITY) {
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[i][c] = 0.f;
            } else {
                corr = expf(m[i] - m_new);
#pragma unroll
                for (int c = 0; c < 4; ++c) { sc[i][c] = expf(sc[i][c] - m_new); psum += sc[i][c]; }
            }
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
            l[i] = l[i] * corr + psum;
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < 4; ++c) Ps[(2 * ry + i) * ldp + cx + 8 * c] = sc[i][c];
            if (cx == 0) cr[2 * ry + i] = corr;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float f = cr[8 * oy + r];
            const f32x2 f2 = pack2(f, f);
#pragma unroll
            for (int k = 0; k < VK; ++k)
#pragma unroll
                for (int c = 0; c < 2; ++c) acc[r][k][c] = mul2(acc[r][k][c], f2);
        }
        for (int c = 0; c < WT_KEYS; ++c) {
            ulonglong2 vv[VK];
#pragma unroll
            for (int k = 0; k < VK; ++k) {
                const int col = 4 * ox + 128 * k;
                vv[k] = col < a.vdim ? *reinterpret_cast<const ulonglong2*>(Vs + c * ldv + col) : make_ulonglong2(0ull, 0ull);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float pv = Ps[(8 * oy + r) * ldp + c];
                const f32x2 p2 = pack2(pv, pv);
#pragma unroll
                for (int k = 0; k < VK; ++k) {
                    acc[r][k][0] = fma2(p2, vv[k].x, acc[r][k][0]);
                    acc[r][k][1] = fma2(p2, vv[k].y, acc[r][k][1]);
                }
            }
        }
    }
    __syncthreads();
    if (cx == 0) {                                     // per row: what its sums are multiplied by at the end
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float f = 1.f / l[i];
            if (a.sink && rv[i]) {
                const float sk = a.sink[g * grp + (2 * ry + i) % grp], mf = fmaxf(m[i], sk), e = expf(m[i] - mf);
                f = e / (l[i] * e + expf(sk - mf));
            }
            cr[2 * ry + i] = f;
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int row = 8 * oy + r;
        if (row >= rows_used) continue;
        const float inv = cr[row];
        float* orow = a.out + ((size_t)(row_base + row / grp) * a.H + g * grp + row % grp) * a.vdim;
#pragma unroll
        for (int k = 0; k < VK; ++k) {
            const int col = 4 * ox + 128 * k;
            if (col < a.vdim) {
                float o0, o1, o2, o3;
                unpack2(acc[r][k][0], o0, o1);
                unpack2(acc[r][k][1], o2, o3);
                *reinterpret_cast<float4*>(orow + col) = make_float4(o0 * inv, o1 * inv, o2 * inv, o3 * inv);
            }
        }
    }
}

// n_single: the step's first rows that are single tokens of running sequences (one CTA per (token, head) each); the prompt
// portions that follow them run on the tiled kernel when the head sizes allow it (multiples of 4, at most 64 query heads
// per key head), otherwise like the single tokens.
int launch_window_attention(const WindowArgs& a, int T, int n_single, const WindowTiles& tm, cudaStream_t stream) {
    FT_REQUIRE(a.H >= 1 && a.G >= 1 && a.H % a.G == 0 && a.dim >= 1 && a.vdim >= 1 && a.vdim <= 512,
               "window attention: bad head sizes (heads %d, kv heads %d, dim %d, vdim %d)", a.H, a.G, a.dim, a.vdim);
    FT_REQUIRE(a.rot_dims >= 0 && a.rot_dims <= a.dim && (a.rot_dims & 1) == 0,
               "window attention: rotary pairs need even sizes (dim %d, rotated %d)", a.dim, a.rot_dims);
    FT_REQUIRE(a.o_v >= 0 || a.v_in_key >= 0 || a.vdim == a.dim || a.no_kv, "window attention: keys used as values need vdim == dim");
    FT_REQUIRE(a.qk_norm >= 0 && a.qk_norm <= 2 && (!a.chunked || a.window > 0), "window attention: bad norm or chunk options");
    FT_REQUIRE(a.keep_first >= 0 && (!a.rel || a.rel_n >= 1) && (a.v_role == 0 || (a.v_first && a.o_v >= 0)) &&
                   (a.v_role != 2 || a.v_mix),
               "window attention: incomplete options");
    window_write_kernel<<<T, 128, a.qk_norm ? (size_t)(a.H + a.G) * 4 : 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    const int grp = a.H / a.G;
    FT_REQUIRE(a.v_in_key < 0 || (a.v_in_key + a.vdim <= a.dim && a.v_role == 0), "window attention: values inside the keys exceed them");
    const size_t tsm = (size_t)((WT_ROWS + 2 * WT_KEYS) * (a.dim + 4) + (a.v_in_key >= 0 ? 0 : 2 * WT_KEYS * a.vdim) + WT_ROWS * (WT_KEYS + 1) + WT_ROWS) * 4;
    const bool tiled = tm.n_tiles > 0 && (a.dim & 3) == 0 && (a.vdim & 3) == 0 && grp <= WT_ROWS && a.vdim <= 256 && tsm <= 220 * 1024 &&
                       (a.v_in_key < 0 || (a.v_in_key & 3) == 0);
    int rows_each = T;                                 // rows of the one-CTA-per-(token, head) kernel
    if (tiled) {
        rows_each = n_single;
        const int QT = WT_ROWS / grp, subs = (64 + QT - 1) / QT;
        dim3 grid(tm.n_tiles * subs, a.G);
        if (a.vdim <= 128) {
            FT_CHECK_CUDA(cudaFuncSetAttribute(window_tile_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsm));
            window_tile_kernel<1><<<grid, WT_THREADS, tsm, stream>>>(a, tm, QT, subs);
        } else {
            FT_CHECK_CUDA(cudaFuncSetAttribute(window_tile_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsm));
            window_tile_kernel<2><<<grid, WT_THREADS, tsm, stream>>>(a, tm, QT, subs);
        }
        FT_CHECK_CUDA(cudaGetLastError());
    }
    if (rows_each <= 0) return 0;
    T = rows_each;
    const size_t smem = (size_t)(((a.dim + 3) & ~3) + 2 * kWinWarps + kWinWarps * a.vdim) * 4;
    const bool vec = (a.dim & 3) == 0 && (a.vdim & 3) == 0;      // every key row then starts on 16 bytes
    dim3 grid(T, a.H);
    const int vpl = (a.vdim + 31) / 32;
#define FT_WIN(V)                                                                                   \
    do {                                                                                            \
        if (vec) window_attn_kernel<V, true><<<grid, kWinWarps * 32, smem, stream>>>(a);            \
        else window_attn_kernel<V, false><<<grid, kWinWarps * 32, smem, stream>>>(a);               \
    } while (0)
    if (vpl <= 1) FT_WIN(1);
    else if (vpl <= 2) FT_WIN(2);
    else if (vpl <= 4) FT_WIN(4);
    else if (vpl <= 8) FT_WIN(8);
    else FT_WIN(16);
#undef FT_WIN
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ scalar-decay rule
// Lanes s = 0..LPC-1 of a column hold channels s * DPT .. s * DPT + DPT - 1 of that column of S.  Chunks of RCH tokens are
// staged in two shared-memory buffers one chunk ahead with asynchronous copies (keys and queries padded with zeros
// to LPC * DPT channels, each lane's run 4 floats apart from the next so that the 16-byte reads of the LPC runs fall into
// different banks), then the tokens of a chunk are taken in order.  A full chunk runs without a branch, so that the
// compiler can start the shared-memory reads of later tokens under the arithmetic of earlier ones, and the arithmetic
// itself is packed: two neighbouring channels of a column share every multiply-add (fma.rn.f32x2, the two-wide fp32
// form of sm_100; each half rounds as the scalar instruction does).  The state is the only dependence from token to token; the
// read-out o_t = S^T q_t (partial sums over a lane's run, then a shuffle tree over the LPC lanes) overlaps the next update.
constexpr int RCH = 16, RTHREADS = 128;
// stages of the ring for a padded row of DP floats: as deep as ~100-160 KB of shared memory allow
__host__ __device__ constexpr int rule_stages(int dp) { return 2; }
template <int N> __device__ __forceinline__ void cp_async_wait_pending() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cp_async_f32(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* dst_smem, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
// VEC: keys and queries are copied 16 bytes at a time (dim a multiple of 4, rows and bases on 16-byte boundaries).
// CPT: state columns per thread.  A thread reads its run of key and query channels once per token and uses it for all of
// its CPT columns — the shared-memory reads, not the arithmetic, bound the kernel with one column per thread (every one of
// a column's 128 / LPC sibling columns in the CTA reads the same runs again).  The CPT partial read-outs are summed over the
// LPC lanes by halving: in each of the first log2(CPT) steps a lane hands half of its columns to its partner and keeps the
// other half, afterwards every lane holds one column and the tree goes on as usual.
template <int LPC, int DPT, int CPT, bool VEC>
__global__ void __launch_bounds__(RTHREADS) decay_rule_kernel(RecurArgs a) {
    constexpr int VB = RTHREADS / LPC * CPT, RUN = DPT + 4, DP = LPC * RUN;
    constexpr int BUF = 2 * RCH * DP + RCH * VB + RCH * 2;      // floats of one staged chunk: keys | queries | values | (a, b)
    constexpr int NST = rule_stages(DP);
    extern __shared__ __align__(16) float rs[];
    const int r = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * VB;
    const int s = threadIdx.x % LPC, jl = threadIdx.x / LPC, j = j0 + jl * CPT;      // the thread's first column
    const int t0 = a.req_start[r], t1 = a.req_start[r + 1];
    if (t1 <= t0) return;
    const int gh = h / (a.heads / a.qk_heads);
    float* S = a.state + (size_t)a.req_slot[r] * a.slot_stride + a.s_off + (size_t)h * a.dim * a.vd;
    if (LPC * DPT != a.dim || j0 + VB > a.vd)                                  // the padding stays zero from here on
        for (int i = threadIdx.x; i < NST * BUF; i += RTHREADS) rs[i] = 0.f;
    f32x2 st[CPT][DPT / 2];                  // per column: channels (2 i, 2 i + 1) of the lane's run
    const bool old = a.req_pos0[r] > 0;
    // four columns of a row are 16 bytes of the state when vd is a multiple of 4 (slots and heads then start on 16 bytes)
    const bool wide = CPT == 4 && (a.vd & 3) == 0 && (((uintptr_t)S) & 15) == 0;
    if (wide) {
#pragma unroll
        for (int i = 0; i < DPT; i += 2) {
            const int d = s * DPT + i;
            float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
            if (old && j < a.vd && d < a.dim) lo = *reinterpret_cast<const float4*>(S + (size_t)d * a.vd + j);
            if (old && j < a.vd && d + 1 < a.dim) hi = *reinterpret_cast<const float4*>(S + (size_t)(d + 1) * a.vd + j);
            const float l4[4] = {lo.x, lo.y, lo.z, lo.w}, h4[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int c = 0; c < CPT; ++c) st[c][i / 2] = pack2(l4[c], h4[c]);
        }
    } else {
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int i = 0; i < DPT; i += 2) {
                const int d = s * DPT + i;
                const bool in = old && j + c < a.vd;
                st[c][i / 2] = pack2(in && d < a.dim ? S[(size_t)d * a.vd + j + c] : 0.f, in && d + 1 < a.dim ? S[(size_t)(d + 1) * a.vd + j + c] : 0.f);
            }
    }
    __syncthreads();
    auto stage = [&](int buf, int c0) {          // always commits a group, an empty one past the end: the count stays uniform
        if (c0 >= t1) { asm volatile("cp.async.commit_group;" ::: "memory"); return; }
        float* sk = rs + buf * BUF;
        float* sq = sk + RCH * DP;
        float* sv = sq + RCH * DP;
        float* sab = sv + RCH * VB;
        const int nt = min(RCH, t1 - c0);
        if (VEC) {                                   // a warp per token row, a lane per four channels
            for (int tt = threadIdx.x >> 5; tt < nt; tt += RTHREADS / 32) {
                const float* kr = a.k + (size_t)(c0 + tt) * a.ldk + (size_t)gh * a.dim;
                const float* qr = a.q + (size_t)(c0 + tt) * a.ldq + (size_t)gh * a.dim;
                for (int d = (threadIdx.x & 31) * 4; d < a.dim; d += 128) {
                    const int at = tt * DP + (d / DPT) * RUN + (d % DPT);
                    cp_async_f32x4(sk + at, kr + d);
                    cp_async_f32x4(sq + at, qr + d);
                }
            }
        } else {
            for (int i = threadIdx.x; i < nt * a.dim; i += RTHREADS) {
                const int tt = i / a.dim, d = i - tt * a.dim;
                const int at = tt * DP + (d / DPT) * RUN + (d % DPT);
                cp_async_f32(sk + at, a.k + (size_t)(c0 + tt) * a.ldk + (size_t)gh * a.dim + d);
                cp_async_f32(sq + at, a.q + (size_t)(c0 + tt) * a.ldq + (size_t)gh * a.dim + d);
            }
        }
        for (int i = threadIdx.x; i < nt * VB; i += RTHREADS) {
            const int tt = i / VB, c = i % VB;
            if (j0 + c < a.vd) cp_async_f32(sv + i, a.v + (size_t)(c0 + tt) * a.ldv + (size_t)h * a.vd + j0 + c);
        }
        for (int i = threadIdx.x; i < nt * 2; i += RTHREADS)
            cp_async_f32(sab + i, a.ab + ((size_t)(c0 + i / 2) * a.heads + h) * 2 + (i & 1));
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < NST - 1; ++i) stage(i, t0 + i * RCH);
    int buf = 0;
    for (int c0 = t0; c0 < t1; c0 += RCH, buf = buf + 1 == NST ? 0 : buf + 1) {
        const int nt = min(RCH, t1 - c0);
        stage(buf == 0 ? NST - 1 : buf - 1, c0 + (NST - 1) * RCH);      // into the buffer the last iteration has finished with
        cp_async_wait_pending<NST - 1>();
        __syncthreads();
        const float* sk = rs + buf * BUF;
        const float* sq = sk + RCH * DP;
        const float* sv = sq + RCH * DP;
        const float* sab = sv + RCH * VB;
        // update: the token's state update and each column's partial read-out over the lane's run
        auto update = [&](int tt, float* o) {
            const float da = sab[2 * tt], db = sab[2 * tt + 1];
            const f32x2 da2 = pack2(da, da);
            f32x2 kk[DPT / 2], qq[DPT / 2];
            const ulonglong2* kp = reinterpret_cast<const ulonglong2*>(sk + tt * DP + s * RUN);
            const ulonglong2* qp = reinterpret_cast<const ulonglong2*>(sq + tt * DP + s * RUN);
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const ulonglong2 kv = kp[i], qv = qp[i];
                kk[2 * i] = kv.x; kk[2 * i + 1] = kv.y;
                qq[2 * i] = qv.x; qq[2 * i + 1] = qv.y;
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float bv = db * sv[tt * VB + jl * CPT + c];
                const f32x2 bv2 = pack2(bv, bv);
                f32x2 o0 = 0ull, o1 = 0ull;
#pragma unroll
                for (int i = 0; i < DPT / 2; i += 2) {
                    st[c][i] = fma2(da2, st[c][i], mul2(bv2, kk[i]));
                    st[c][i + 1] = fma2(da2, st[c][i + 1], mul2(bv2, kk[i + 1]));
                    o0 = fma2(st[c][i], qq[i], o0);
                    o1 = fma2(st[c][i + 1], qq[i + 1], o1);
                }
                float p0, p1, p2, p3;
                unpack2(o0, p0, p1);
                unpack2(o1, p2, p3);
                o[c] = (p0 + p2) + (p1 + p3);
            }
        };
        // finish: sum over the LPC lanes; the column a lane ends up with is made of the lane bits used in the halving steps.
        // Taken for four tokens at a time, so that the shuffle chains of the four overlap instead of stalling the warp.
        auto finish = [&](int tt, const float* o) {
            int col = 0;
            float v = o[0];
            if (CPT == 4) {
                const bool up = (s & (LPC / 2)) != 0, up2 = (s & (LPC / 4)) != 0;
                const float g0 = __shfl_xor_sync(0xffffffffu, up ? o[0] : o[2], LPC / 2);
                const float g1 = __shfl_xor_sync(0xffffffffu, up ? o[1] : o[3], LPC / 2);
                const float k0 = (up ? o[2] : o[0]) + g0, k1 = (up ? o[3] : o[1]) + g1;
                const float g2 = __shfl_xor_sync(0xffffffffu, up2 ? k0 : k1, LPC / 4);
                v = (up2 ? k1 : k0) + g2;
                col = (up ? 2 : 0) + (up2 ? 1 : 0);
#pragma unroll
                for (int off = LPC / 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            } else if (CPT == 2) {
                const bool up = (s & (LPC / 2)) != 0;
                const float g0 = __shfl_xor_sync(0xffffffffu, up ? o[0] : o[1], LPC / 2);
                v = (up ? o[1] : o[0]) + g0;
                col = up ? 1 : 0;
#pragma unroll
                for (int off = LPC / 4; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            } else {
#pragma unroll
                for (int off = LPC / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            }
            if ((s & (LPC / CPT - 1)) == 0 && j + col < a.vd) a.o[(size_t)(c0 + tt) * a.ldo + (size_t)h * a.vd + j + col] = v;
        };
        if (nt == RCH) {
#pragma unroll 1
            for (int t4 = 0; t4 < RCH; t4 += 4) {
                float o[4][CPT];
#pragma unroll
                for (int x = 0; x < 4; ++x) update(t4 + x, o[x]);
#pragma unroll
                for (int x = 0; x < 4; ++x) finish(t4 + x, o[x]);
            }
        } else {
            for (int tt = 0; tt < nt; ++tt) {
                float o[CPT];
                update(tt, o);
                finish(tt, o);
            }
        }
        __syncthreads();
    }
    if (wide) {
#pragma unroll
        for (int i = 0; i < DPT; i += 2) {
            const int d = s * DPT + i;
            float l4[4], h4[4];
#pragma unroll
            for (int c = 0; c < CPT; ++c) unpack2(st[c][i / 2], l4[c], h4[c]);
            if (j < a.vd && d < a.dim) *reinterpret_cast<float4*>(S + (size_t)d * a.vd + j) = make_float4(l4[0], l4[1], l4[2], l4[3]);
            if (j < a.vd && d + 1 < a.dim) *reinterpret_cast<float4*>(S + (size_t)(d + 1) * a.vd + j) = make_float4(h4[0], h4[1], h4[2], h4[3]);
        }
        return;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < DPT; i += 2) {
            const int d = s * DPT + i;
            float lo, hi;
            unpack2(st[c][i / 2], lo, hi);
            if (j + c < a.vd && d < a.dim) S[(size_t)d * a.vd + j + c] = lo;
            if (j + c < a.vd && d + 1 < a.dim) S[(size_t)(d + 1) * a.vd + j + c] = hi;
        }
}

template <int LPC, int DPT, int CPT>
static int launch_decay_rule_t(const RecurArgs& a, int n_req, cudaStream_t stream) {
    constexpr int VB = RTHREADS / LPC * CPT, DP = LPC * (DPT + 4);
    const size_t smem = (size_t)rule_stages(DP) * (2 * RCH * DP + RCH * VB + RCH * 2) * 4;
    const bool vec = (a.dim & 3) == 0 && (a.ldk & 3) == 0 && (a.ldq & 3) == 0 && ((uintptr_t)a.k & 15) == 0 && ((uintptr_t)a.q & 15) == 0;
    if (smem > 48 * 1024) {
        FT_CHECK_CUDA(cudaFuncSetAttribute(decay_rule_kernel<LPC, DPT, CPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FT_CHECK_CUDA(cudaFuncSetAttribute(decay_rule_kernel<LPC, DPT, CPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    dim3 grid((a.vd + VB - 1) / VB, a.heads, n_req);
    if (vec) decay_rule_kernel<LPC, DPT, CPT, true><<<grid, RTHREADS, smem, stream>>>(a);
    else decay_rule_kernel<LPC, DPT, CPT, false><<<grid, RTHREADS, smem, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// Lanes per column (LPC), channels per lane (DPT <= 16, 32 only beyond 512 channels) and columns per thread (CPT): the
// fewest lanes whose runs cover dim and four columns per thread — the widest column blocks, the best-coalesced state
// traffic and the fewest shared-memory reads per multiply-add; then, while fewer than 96 CTAs would run (one long prompt
// with few heads): two columns per thread, more lanes with shorter runs, at last one column (measured order).  The split
// changes the order of a sum, nothing else.  a.lanes fixes LPC.  T: tokens in the step (unused by the present rule, kept
// for callers that tune).
int launch_decay_rule(const RecurArgs& a, int n_req, int T, cudaStream_t stream) {
    (void)T;
    FT_REQUIRE(a.heads >= 1 && a.qk_heads >= 1 && a.heads % a.qk_heads == 0 && a.dim >= 1 && a.dim <= 1024 && a.vd >= 1,
               "decay rule: bad sizes (heads %d, key heads %d, dim %d, values %d)", a.heads, a.qk_heads, a.dim, a.vd);
    if (n_req <= 0) return 0;
    int lpc = 4, dpt = 4;
    while (dpt < 16 && lpc * dpt < a.dim) dpt *= 2;
    while (lpc < 32 && lpc * dpt < a.dim) lpc *= 2;
    if (lpc * dpt < a.dim) dpt = 32;
    int cpt = dpt == 32 ? 2 : 4;
    auto ctas = [&](int l, int c) { return (long long)n_req * a.heads * ((a.vd + RTHREADS / l * c - 1) / (RTHREADS / l * c)); };
    if (a.lanes > 0) {
        FT_REQUIRE((a.lanes == 4 || a.lanes == 8 || a.lanes == 16 || a.lanes == 32) && a.lanes >= lpc,
                   "decay rule: %d lanes per column do not hold %d channels", a.lanes, a.dim);
        while (lpc < a.lanes && dpt > 4) { lpc *= 2; dpt /= 2; }
        cpt = dpt == 32 ? 2 : 4;
        while (cpt > 1 && ctas(lpc, cpt) < 96) cpt /= 2;
    } else {
        while (ctas(lpc, cpt) < 96) {
            if (cpt > 2) cpt = 2;
            else if (lpc < 32 && dpt > 4) { lpc *= 2; dpt /= 2; }
            else if (cpt > 1) cpt = 1;
            else break;
        }
    }
#define FT_RULE(L, D, C) if (lpc == L && dpt == D && cpt == C) return launch_decay_rule_t<L, D, C>(a, n_req, stream)
#define FT_RULE_L(L) FT_RULE(L, 4, 1); FT_RULE(L, 4, 2); FT_RULE(L, 4, 4); FT_RULE(L, 8, 1); FT_RULE(L, 8, 2); FT_RULE(L, 8, 4); \
                     FT_RULE(L, 16, 1); FT_RULE(L, 16, 2); FT_RULE(L, 16, 4)
    FT_RULE_L(4); FT_RULE_L(8); FT_RULE_L(16); FT_RULE_L(32);
    FT_RULE(32, 32, 1); FT_RULE(32, 32, 2);
#undef FT_RULE_L
#undef FT_RULE
    FT_REQUIRE(false, "decay rule: no kernel for %d lanes x %d channels x %d columns", lpc, dpt, cpt);
    return -1;
}

extern "C" int ft_decay_rule(const float* q, const float* k, const float* v, const float* ab, float* o, float* state,
                             const int* req_start, const int* req_pos0, const int* req_slot, int n_req, int heads, int qk_heads,
                             int dim, int vd, long long slot_stride, int lanes, int T, void* stream) {
    FT_REQUIRE(q && k && v && ab && o && state && req_start && req_pos0 && req_slot, "ft_decay_rule: null argument");
    RecurArgs a;
    a.q = q; a.k = k; a.v = v; a.ab = ab; a.o = o; a.state = state;
    a.ldq = a.ldk = qk_heads * dim; a.ldv = a.ldo = heads * vd;
    a.slot_stride = slot_stride; a.s_off = 0;
    a.req_start = req_start; a.req_pos0 = req_pos0; a.req_slot = req_slot;
    a.heads = heads; a.qk_heads = qk_heads; a.dim = dim; a.vd = vd; a.lanes = lanes;
    return launch_decay_rule(a, n_req, T, (cudaStream_t)stream);
}

// ------------------------------------------------------------------ gated matrix memory: gates and the running maximum
// Per token: values with a column of ones appended (the normaliser rides along as one more state column), and the log
// gates i = cap tanh((z_i + b_i) / cap), f = logsigmoid(cap tanh((z_f + b_f) / cap)).
__global__ void __launch_bounds__(128) memory_prep_kernel(MemoryArgs a) {
    const int t = blockIdx.x;
    const float* pr = a.proj + (size_t)t * a.ldp;
    const int ve = a.vdim + 1;
    for (int i = threadIdx.x; i < a.heads * ve; i += blockDim.x) {
        const int h = i / ve, j = i % ve;
        a.v_ext[(size_t)t * a.heads * ve + i] = j < a.vdim ? pr[a.o_v + h * a.vdim + j] : 1.f;
    }
    for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
        const float zi = pr[a.o_i + h] + a.gate_bias[h], zf = pr[a.o_f + h] + a.gate_bias[a.heads + h];
        const float gi = a.cap * tanhf(zi / a.cap);
        const float gf = -softplus_f(-(a.cap * tanhf(zf / a.cap)));
        a.gates[((size_t)t * a.heads + h) * 2] = gi;
        a.gates[((size_t)t * a.heads + h) * 2 + 1] = gf;
    }
}
// One warp per (request, head): m_t = max(f_t + m_(t-1), i_t) is a scan under the associative rule
// (F1, G1) o (F2, G2) = (F1 + F2, max(G1 + F2, G2)), so 32 tokens are taken at a time with shuffles and m enters each block as
// m_t = max(F_t + m_in, G_t).  Then a = exp(f + m_(t-1) - m_t), b = exp(i - m_t), floor[t] = exp(-m_t), the lower bound of the
// read-out's denominator.  m lives in the state slot, 0 at a sequence's start.
__global__ void __launch_bounds__(128) memory_scan_kernel(MemoryArgs a, int n_units) {
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= n_units) return;
    const int r = unit / a.heads, h = unit % a.heads;
    const int t0 = a.req_start[r], t1 = a.req_start[r + 1];
    if (t1 <= t0) return;
    float* ms = a.state + (size_t)a.req_slot[r] * a.slot_stride + a.m_off + h;
    float m = a.req_pos0[r] > 0 ? *ms : 0.f;
    for (int b0 = t0; b0 < t1; b0 += 32) {
        const int t = b0 + lane;
        const bool in = t < t1;
        const size_t at = (size_t)(in ? t : t1 - 1) * a.heads + h;
        const float gi = in ? a.gates[2 * at] : -INFINITY, gf = in ? a.gates[2 * at + 1] : 0.f;
        float F = gf, G = gi;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float pF = __shfl_up_sync(0xffffffffu, F, off), pG = __shfl_up_sync(0xffffffffu, G, off);
            if (lane >= off) { G = fmaxf(pG + F, G); F = pF + F; }
        }
        const float mt = fmaxf(F + m, G);
        float mp = __shfl_up_sync(0xffffffffu, mt, 1);
        if (lane == 0) mp = m;
        if (in) {
            a.ab[2 * at] = expf(gf + mp - mt);
            a.ab[2 * at + 1] = expf(gi - mt);
            a.floor[at] = expf(-mt);
        }
        m = __shfl_sync(0xffffffffu, mt, min(31, t1 - 1 - b0));
    }
    if (lane == 0) *ms = m;
}
int launch_memory_prep(const MemoryArgs& a, int T, int n_req, cudaStream_t stream) {
    FT_REQUIRE(a.heads >= 1 && a.cap > 0.f, "matrix memory: bad head count or gate cap");
    memory_prep_kernel<<<T, 128, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    const int units = n_req * a.heads;
    memory_scan_kernel<<<(units + 3) / 4, 128, 0, stream>>>(a, units);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ state space: convolution, step sizes, tails
// u = raw x | B | C channels of a token (proj columns o_x ..).  out[t][c] = silu(bias[c] + sum_j w[c][K-1-j] u[t-j][c]); rows
// before the step's first come from the slot's tail (the last K-1 raw inputs of the sequence), zeros before position 0.
__global__ void __launch_bounds__(256) space_conv_kernel(SpaceArgs a) {
    const int t = blockIdx.x;
    const int r = a.seq_rows[t];
    const int start = a.req_start[r], pos0 = a.req_pos0[r], K = a.taps;
    const int k = t - start;
    const float* tail = a.state + (size_t)a.req_slot[r] * a.slot_stride + a.tail_off;
    for (int c = threadIdx.x; c < a.channels; c += blockDim.x) {
        float acc = a.conv_b ? a.conv_b[c] : 0.f;
        for (int j = 0; j < K; ++j) {
            float u = 0.f;
            if (k - j >= 0) u = a.proj[(size_t)(t - j) * a.ldp + a.o_x + c];
            else if (pos0 + k - j >= 0) u = tail[(size_t)c * (K - 1) + (k - j + K - 1)];
            acc = fmaf(a.conv_w[(size_t)c * K + (K - 1 - j)], u, acc);
        }
        a.xbc[(size_t)t * a.channels + c] = a.act ? silu_f(acc) : acc;
    }
    for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
        const float dt = softplus_f(a.proj[(size_t)t * a.ldp + a.o_dt + h] + a.dt_bias[h]);
        a.ab[((size_t)t * a.heads + h) * 2] = expf(-expf(a.a_log[h]) * dt);
        a.ab[((size_t)t * a.heads + h) * 2 + 1] = dt;
    }
}
// The slot's tail after the step: the raw inputs of the last K-1 positions, from this step's rows or the old tail.
constexpr int kMaxTaps = 16;
__global__ void __launch_bounds__(256) space_tail_kernel(SpaceArgs a) {
    const int r = blockIdx.y;
    const int start = a.req_start[r], n = a.req_start[r + 1] - start, pos0 = a.req_pos0[r], K = a.taps;
    if (n <= 0 || K <= 1) return;
    float* tail = a.state + (size_t)a.req_slot[r] * a.slot_stride + a.tail_off;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < a.channels; c += gridDim.x * blockDim.x) {
        float nv[kMaxTaps];
        for (int i = 0; i < K - 1; ++i) {
            const int k = n - (K - 1) + i;
            float u = 0.f;
            if (k >= 0) u = a.proj[(size_t)(start + k) * a.ldp + a.o_x + c];
            else if (pos0 + k >= 0) u = tail[(size_t)c * (K - 1) + (k + K - 1)];
            nv[i] = u;
        }
        for (int i = 0; i < K - 1; ++i) tail[(size_t)c * (K - 1) + i] = nv[i];
    }
}
int launch_space_prep(const SpaceArgs& a, int T, int n_req, cudaStream_t stream) {
    FT_REQUIRE(a.taps >= 1 && a.taps <= kMaxTaps, "state space: 1 to %d convolution taps (got %d)", kMaxTaps, a.taps);
    space_conv_kernel<<<T, 256, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    space_tail_kernel<<<dim3((a.channels + 255) / 256, n_req), 256, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ read-out of the recurrent branches
// One CTA per (token, norm group).  Value of column c = (head h, j):
//   o[t][h * vd + j] * q_scale                              (vd = vdim, or vdim + 1 with the normaliser in the last column)
//   / (max(|o[t][h * vd + vdim] * q_scale|, floor[t][h]) + 1e-6)      with a normaliser
//   + skip[h] * x[t][c]                                      with a skip
//   * silu(gate[t][c])                                       gate_kind 1 (before the norm)
// then divided by the root mean square of its group, times gain[c], times sigmoid(gate[t][c]) for gate_kind 2.
__device__ __forceinline__ float readout_value(const ReadoutArgs& a, int t, int c) {
    const int h = c / a.vdim, j = c % a.vdim;
    const float* orow = a.o + (size_t)t * a.ldo + (size_t)h * a.vd;
    float v = orow[j] * a.q_scale;
    if (a.floor) v = v / (fmaxf(fabsf(orow[a.vdim] * a.q_scale), a.floor[(size_t)t * a.heads + h]) + 1e-6f);
    if (a.skip) v = fmaf(a.skip[h], a.x[(size_t)t * a.ldx + c], v);
    if (a.gate_kind == 1) v *= silu_f(a.gate[(size_t)t * a.ldg + c]);
    return v;
}
constexpr int kReadoutKeep = 8;      // values a thread keeps in registers between the two passes
__global__ void __launch_bounds__(256) readout_kernel(ReadoutArgs a) {
    __shared__ float red[33];
    const int t = blockIdx.x / a.norm_groups, g = blockIdx.x % a.norm_groups;
    const int n = a.heads * a.vdim / a.norm_groups, c0 = g * n;
    float keep[kReadoutKeep];
    float ss = 0.f;
    int i = 0;
    for (int c = threadIdx.x; c < n; c += blockDim.x, ++i) {
        const float v = readout_value(a, t, c0 + c);
        if (i < kReadoutKeep) keep[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = blockDim.x == 32 ? warp_sum(ss) : cta_sum(ss, red);
    const float rr = 1.f / sqrtf(ss / (float)n + a.eps);
    i = 0;
    for (int c = threadIdx.x; c < n; c += blockDim.x, ++i) {
        float v = (i < kReadoutKeep ? keep[i] : readout_value(a, t, c0 + c)) * rr * a.gain[c0 + c];
        if (a.gate_kind == 2) v *= sigmoid_f(a.gate[(size_t)t * a.ldg + c0 + c]);
        a.out[(size_t)t * a.heads * a.vdim + c0 + c] = v;
    }
}
int launch_readout(const ReadoutArgs& a, int T, cudaStream_t stream) {
    FT_REQUIRE(a.norm_groups >= 1 && (a.heads * a.vdim) % a.norm_groups == 0, "read-out: %d columns do not split into %d norm groups",
               a.heads * a.vdim, a.norm_groups);
    const int n = a.heads * a.vdim / a.norm_groups;
    const int threads = n <= 64 ? 32 : n <= 256 ? 64 : n <= 1024 ? 128 : 256;
    readout_kernel<<<T * a.norm_groups, threads, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ activations between the two halves of a feed-forward
// SwiGLU: gu [rows][2 ff] with columns (2j, 2j+1) = (gate_j, up_j) -> out [rows][ff]; squared ReLU: [rows][ff] -> [rows][ff]
__global__ void ff_act_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n, int act) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        if (act == FT_ACT_RELU2) { const float v = fmaxf(in[i], 0.f); out[i] = v * v; }
        else { const float2 v = reinterpret_cast<const float2*>(in)[i]; out[i] = silu_f(v.x) * v.y; }
    }
}
int launch_ff_act(const float* in, float* out, size_t n, int act, cudaStream_t stream) {
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
    ff_act_kernel<<<blocks, 256, 0, stream>>>(in, out, n, act);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace ft
