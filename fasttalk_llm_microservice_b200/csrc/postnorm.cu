// Kernels of the post-norm layer form (FT_LAYER_POSTNORM) and the staging of latent window attention.  Everything fp32.
//
//   embedding            x = embed[token] * scale, also kept as X_0 of the depth history
//   input convolution    what a sublayer reads: hn = x + conv(x), a causal convolution over time per coordinate whose
//                        inputs before the step's first row come from the slot's ring of stream rows
//   post norm            x += rms(y) * gain for a sublayer's result y (one or two branch results with their biases), fused
//                        with what follows it: the ring's new rows, and either the next sublayer's input convolution or, at a
//                        layer's end, the weighted sum over depth (the new row is X_k, the stream becomes sum_j w_j X_j)
//   row norms            the model's last norm over the wanted rows; a run of columns normed to a place (latents)
#include "common.cuh"
#include "ft_internal.h"

namespace ft {

namespace {
__device__ __forceinline__ float block_sum(float v, float* red) {      // red: >= 33 floats of shared memory
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
__device__ __forceinline__ void planes_put(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t i, float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
}
}  // namespace

__global__ void __launch_bounds__(256)
embed_scale_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed, float scale, float* __restrict__ x,
                   float* __restrict__ hist, int W) {
    const int t = blockIdx.x;
    const __nv_bfloat16* e = embed + (size_t)tokens[t] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = __bfloat162float(e[c]) * scale;
        x[(size_t)t * W + c] = v;
        if (hist) hist[(size_t)t * W + c] = v;
    }
}
int launch_embed_scale(const int* tokens, const void* embed, float scale, float* x, float* hist, int T, int W, cudaStream_t stream) {
    embed_scale_kernel<<<T, 256, 0, stream>>>(tokens, (const __nv_bfloat16*)embed, scale, x, hist, W);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ input convolution
// The rows a convolution needs from before the step live in the session's slot as a ring over positions: the stream row of
// position p (as the sublayer saw it) sits in ring[p % (taps - 1)].  The ring is READ by the kernel that forms the
// sublayer's input and WRITTEN by the post-norm kernel that follows the sublayer (it still holds the rows the sublayer read):
// two launches in stream order, so a step never reads a ring entry that it has already replaced.
constexpr int kCanonMaxTaps = 17;
__global__ void __launch_bounds__(256) canon_kernel(CanonArgs a) {
    const int t = blockIdx.x, W = a.W, taps = a.taps, keep = taps - 1;
    const int req = a.seq_rows[t];
    const int r = t - a.req_start[req];              // index inside this step's portion
    const int pos0 = a.req_pos0[req];
    const float* ring = a.state + (size_t)a.req_slot[req] * a.slot_stride + a.tail_off;      // [taps - 1][W]
    __nv_bfloat16 *hi = (__nv_bfloat16*)a.hi, *lo = (__nv_bfloat16*)a.lo;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float s = a.x[(size_t)t * W + c];
        if (a.w) {
            float acc = 0.f;
            for (int i = 0; i < taps; ++i) {
                const int back = taps - 1 - i;
                float v;
                if (r - back >= 0) v = a.x[(size_t)(t - back) * W + c];
                else if (pos0 + r - back >= 0) v = ring[(size_t)((pos0 + r - back) % keep) * W + c];
                else v = 0.f;
                acc = fmaf(a.w[(size_t)c * taps + i], v, acc);
            }
            s += acc;
        }
        a.hn[(size_t)t * W + c] = s;
        if (hi) planes_put(hi, lo, (size_t)t * W + c, s);
    }
}
int launch_canon(const CanonArgs& a, int T, cudaStream_t stream) {
    FT_REQUIRE(a.x && a.hn && a.W >= 1, "input convolution: missing operands");
    FT_REQUIRE(!a.w || (a.taps >= 1 && a.taps <= kCanonMaxTaps && a.state), "input convolution: %d taps are beyond %d", a.taps,
               kCanonMaxTaps);
    canon_kernel<<<T, 256, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ post norm, the sum over depth, the next input
// One kernel per sublayer joint, one CTA per row t:
//   (1) the row the sublayer read goes into its ring when it is among the last taps - 1 of its sequence in this step;
//   (2) v = x[t] + rms(y[t]) * post_w;
//   (3) at a layer's end: hist[k][t] = v and the stream becomes sum_j depth_w[j] hist[j][t];
//   (4) otherwise, with cw: the NEXT sublayer's input hn[t] = v + sum_i cw[:, i] v[t - taps + 1 + i].  The earlier rows of
//       the step are formed again from their own x and y (a row's norm needs nothing but that row), rows before the step
//       come from the next sublayer's ring.  The new rows go to x_out, a buffer of its own, since the CTAs of the following
//       rows read the old x[t].
__device__ __forceinline__ float post_y(const PostNormArgs& a, size_t i, int c) {
    float y = a.y0[i] + (a.b0 ? a.b0[c] : 0.f);
    if (a.y1) y = a.s0 * y + a.s1 * (a.y1[i] + (a.b1 ? a.b1[c] : 0.f));
    else if (a.s0 != 1.f) y *= a.s0;
    return y;
}
__global__ void __launch_bounds__(256) postnorm_kernel(PostNormArgs a) {
    __shared__ float red[33];
    extern __shared__ float sm[];
    const int t = blockIdx.x, W = a.W;
    float* row = sm;                                  // [W] y of the row at hand
    float* acc = sm + W;                              // [W] the convolution's sum (only with cw)
    int r = 0, pos0 = 0, n = 1;
    float* slot = nullptr;
    if (a.seq_rows) {
        const int req = a.seq_rows[t];
        r = t - a.req_start[req];
        n = a.req_start[req + 1] - a.req_start[req];
        pos0 = a.req_pos0[req];
        slot = a.state + (size_t)a.req_slot[req] * a.slot_stride;
    }
    const int keep = a.taps - 1;
    if (a.save_off >= 0 && keep > 0 && r >= n - keep) {
        float* ring = slot + a.save_off + (size_t)((pos0 + r) % keep) * W;
        for (int c = threadIdx.x; c < W; c += blockDim.x) ring[c] = a.x[(size_t)t * W + c];
    }
    const int first = a.cw ? keep : 0;                // how many earlier rows are formed again
    if (a.cw)
        for (int c = threadIdx.x; c < W; c += blockDim.x) acc[c] = 0.f;
    for (int b = first; b >= 0; --b) {
        const int rb = r - b;                         // uniform over the CTA
        const float* cwb = a.cw ? a.cw + (a.taps - 1 - b) : nullptr;
        if (rb < 0) {
            if (pos0 + rb < 0) continue;
            const float* ring = slot + a.read_off + (size_t)((pos0 + rb) % keep) * W;
            for (int c = threadIdx.x; c < W; c += blockDim.x) acc[c] = fmaf(cwb[(size_t)c * a.taps], ring[c], acc[c]);
            continue;
        }
        const size_t base = (size_t)(t - b) * W;
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float y = post_y(a, base + c, c);
            row[c] = y;
            ss += y * y;
        }
        ss = block_sum(ss, red);
        const float rs = 1.f / sqrtf(ss / (float)W + a.eps);
        if (b > 0) {
            for (int c = threadIdx.x; c < W; c += blockDim.x)
                acc[c] = fmaf(cwb[(size_t)c * a.taps], a.x[base + c] + row[c] * rs * a.post_w[c], acc[c]);
            continue;
        }
        __nv_bfloat16 *hi = (__nv_bfloat16*)a.hi, *lo = (__nv_bfloat16*)a.lo;
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            float v = a.x[base + c] + row[c] * rs * a.post_w[c];
            if (a.hist) {
                a.hist[((size_t)a.k * a.t_stride + t) * W + c] = v;
                if (a.depth_w) {
                    v *= a.depth_w[a.k];
                    for (int j = a.k - 1; j >= 0; --j) v = fmaf(a.depth_w[j], a.hist[((size_t)j * a.t_stride + t) * W + c], v);
                }
            }
            a.x_out[base + c] = v;
            if (a.cw) {
                const float h = v + fmaf(cwb[(size_t)c * a.taps], v, acc[c]);
                a.hn[base + c] = h;
                if (hi) planes_put(hi, lo, base + c, h);
            }
        }
    }
}
int launch_postnorm(const PostNormArgs& a, int T, cudaStream_t stream) {
    FT_REQUIRE(a.x && a.x_out && a.y0 && a.post_w && a.W >= 1, "post norm: missing operands");
    FT_REQUIRE(!a.cw || (a.x_out != a.x && a.hn && !a.hist && a.taps >= 1 && a.taps <= kCanonMaxTaps && (a.taps == 1 || a.seq_rows)),
               "post norm: the fused input convolution needs a second stream buffer and the step's rows");
    FT_REQUIRE(a.save_off < 0 || a.taps <= 1 || a.seq_rows, "post norm: saving rows needs the step's rows");
    postnorm_kernel<<<T, 256, (size_t)a.W * 8, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ row norms
__global__ void __launch_bounds__(256)
rms_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w, float gain,
                float* __restrict__ out, int W, float eps) {
    __shared__ float red[33];
    const float* src = x + (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss += src[c] * src[c];
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[(size_t)blockIdx.x * W + c] = src[c] * r * (w ? w[c] : gain);
}
int launch_rms_rows(const float* x, const int* rows, const float* w, float gain, float* out, int n, int W, float eps,
                    cudaStream_t stream) {
    rms_rows_kernel<<<n, 256, 0, stream>>>(x, rows, w, gain, out, W, eps);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

__global__ void __launch_bounds__(128)
rms_cols_kernel(const float* __restrict__ src, int lds, int src_off, const float* __restrict__ w, float* __restrict__ dst, int ldd,
                int dst_off, int n, float eps) {
    __shared__ float red[33];
    const float* s = src + (size_t)blockIdx.x * lds + src_off;
    float* d = dst + (size_t)blockIdx.x * ldd + dst_off;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) ss += s[c] * s[c];
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) d[c] = s[c] * r * w[c];
}
int launch_rms_cols(const float* src, int lds, int src_off, const float* w, float* dst, int ldd, int dst_off, int n, float eps,
                    int T, cudaStream_t stream) {
    rms_cols_kernel<<<T, 128, 0, stream>>>(src, lds, src_off, w, dst, ldd, dst_off, n, eps);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// Latent window attention, per token: from the query projection q [heads][dim plain | rot] and the layer's projection
// (kv_rank latent columns, then rot columns of the shared key part at o_k) to the staging row the window-attention kernels read:
//   [heads x (rot query part | folded plain query, written by the caller's GEMM)] [rot key part | normed latent]
__global__ void __launch_bounds__(128)
latent_stage_kernel(const float* __restrict__ q, int heads, int dim, int rot, const float* __restrict__ proj, int ldp, int o_k,
                    int rank, const float* __restrict__ w, float eps, float* __restrict__ stage, int lds) {
    __shared__ float red[33];
    const int t = blockIdx.x, kd = rot + rank;
    float* st = stage + (size_t)t * lds;
    const float* qr = q + (size_t)t * heads * (dim + rot);
    for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
        const int h = i / rot, c = i - h * rot;
        st[(size_t)h * kd + c] = qr[(size_t)h * (dim + rot) + dim + c];
    }
    const float* pr = proj + (size_t)t * ldp + o_k;
    float* key = st + (size_t)heads * kd;
    for (int c = threadIdx.x; c < rot; c += blockDim.x) key[c] = pr[rank + c];
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) ss += pr[c] * pr[c];
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)rank + eps);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = pr[c] * r * w[c];
        key[rot + c] = v;
    }
}
int launch_latent_stage(const float* q, int heads, int dim, int rot, const float* proj, int ldp, int o_k, int rank, const float* w,
                        float eps, float* stage, int lds, int T, cudaStream_t stream) {
    latent_stage_kernel<<<T, 128, 0, stream>>>(q, heads, dim, rot, proj, ldp, o_k, rank, w, eps, stage, lds);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace ft
