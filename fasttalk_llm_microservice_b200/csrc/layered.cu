// Kernels of the layered model family: decoders described layer by layer (ft_layer_desc), whose sizes are all run-time
// values.  The residual stream, the normed layer input, every projection output, attention scores and weights, router
// scores and the recurrent state are fp32; weights are bf16 and are multiplied as the fp32 numbers they are, with fp32
// accumulation in a fixed order per output element — a row's result does not depend on which other rows share its launch.
//
//   linear              C[r, n] = sum_k A[row(r), k] * W[p][n, k]: plain, batched over heads (column offsets per problem)
//                       or grouped over experts (row segments per problem, rows gathered through an index list), with
//                       fused epilogues (paired SwiGLU, tanh soft cap); a 64 x 64 tile kernel for many rows and a
//                       warp-per-output kernel for a handful of rows (decode)
//   embed / combine     embedding gather; gated-residual update of the stream, both fused with the scalar-gain RMS norm
//                       of the next layer
//   latent attention    the latent of every token is normed and written to a paged fp32 cache; queries are folded into
//                       latent space (q W_uk), scores, softmax and the weighted sum run over the cached latents, values
//                       are expanded afterwards (W_uv): only the latent is ever stored
//   channel delta       short causal convolutions + SiLU + unit norms + per-channel decays, then the gated delta rule
//                       token by token with one thread per state column, state and convolution tails in per-session slots
//   router              softmax over all experts, group-limited top-k, counting sort of (token, choice) pairs by expert
#include "common.cuh"
#include "ft_internal.h"

#include <algorithm>

namespace ft {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_exact(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float bf16_to_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }

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

// asynchronous global -> shared copies (the staging of the delta rule and of the tensor-core attention)
__device__ __forceinline__ void cp_async4(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ------------------------------------------------------------------ linear: tile kernel
constexpr int LBM = 64, LBN = 64, LBK = 16, LTHREADS = 256;

template <bool VEC>
__global__ void __launch_bounds__(LTHREADS) linear_tile_kernel(LinearArgs a) {
    __shared__ float sA[LBK][LBM + 4];
    __shared__ float sW[LBK][LBN + 4];
    __shared__ int s_info[3];
    int p, row0, rows_end;
    if (a.seg) {                       // grouped: blockIdx.y enumerates the row tiles of all segments
        if (threadIdx.x == 0) {
            int tile = blockIdx.y, pp = 0, found = -1, r0 = 0, r1 = 0;
            for (; pp < a.P; ++pp) {
                const int s0 = a.seg[pp], s1 = a.seg[pp + 1];
                const int nt = (s1 - s0 + LBM - 1) / LBM;
                if (tile < nt) { found = pp; r0 = s0 + tile * LBM; r1 = s1; break; }
                tile -= nt;
            }
            s_info[0] = found; s_info[1] = r0; s_info[2] = r1;
        }
        __syncthreads();
        p = s_info[0]; row0 = s_info[1]; rows_end = s_info[2];
        if (p < 0) return;
    } else {
        p = blockIdx.z; row0 = blockIdx.y * LBM; rows_end = a.M;
    }
    const int n0 = blockIdx.x * LBN;
    const float* A = a.A + (size_t)p * a.a_col_stride;
    const __nv_bfloat16* W = a.W + (size_t)p * a.w_stride;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 16 x 16 threads, 4 x 4 outputs each
    // Every output is summed in two levels: the LBK products of a K tile in one short chain, the tiles' sums with a running
    // compensation term (the rounding error of each addition is carried into the next), so the result's error does not grow
    // with K as one long chain of multiply-adds would.
    float acc[4][4], comp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = comp[i][j] = 0.f;
    // loader mapping: thread -> (row within tile, 4 consecutive k)
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    const int arow_t = row0 + lr;
    long long arow = -1;
    if (arow_t < rows_end) arow = a.a_rows ? a.a_rows[arow_t] : arow_t;
    const int wrow = n0 + lr;
    for (int k0 = 0; k0 < a.K; k0 += LBK) {
        float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + lk;
        if (arow >= 0) {
            const float* ap = A + arow * a.lda + k;
            if (VEC && k + 3 < a.K) {
                const float4 t = *reinterpret_cast<const float4*>(ap);
                av[0] = t.x; av[1] = t.y; av[2] = t.z; av[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < a.K) av[i] = ap[i];
            }
        }
        if (wrow < a.N) {
            const __nv_bfloat16* wp = W + (size_t)wrow * a.ldw + k;
            if (VEC && k + 3 < a.K) {
                const uint2 t = *reinterpret_cast<const uint2*>(wp);
                wv[0] = bf16_lo(t.x); wv[1] = bf16_hi(t.x); wv[2] = bf16_lo(t.y); wv[3] = bf16_hi(t.y);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < a.K) wv[i] = __bfloat162float(wp[i]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) { sA[lk + i][lr] = av[i]; sW[lk + i][lr] = wv[i]; }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < LBK; ++kk) {
            const float4 x = *reinterpret_cast<const float4*>(&sA[kk][ty * 4]);
            const float4 w = *reinterpret_cast<const float4*>(&sW[kk][tx * 4]);
            const float xa[4] = {x.x, x.y, x.z, x.w}, wa[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(xa[i], wa[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float y = part[i][j] - comp[i][j];
                const float t = __fadd_rn(acc[i][j], y);
                comp[i][j] = __fadd_rn(__fadd_rn(t, -acc[i][j]), -y);
                acc[i][j] = t;
            }
    }
    float* C = a.C + (size_t)p * a.c_col_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= rows_end) continue;
        if (a.epi == LIN_SWIGLU_PAIR) {          // columns (2j, 2j+1) = (gate_j, up_j) -> C[r, j]
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < a.N) {
                    const float g = acc[i][j];
                    C[(size_t)r * a.ldc + (n >> 1)] = g / (1.f + expf(-g)) * acc[i][j + 1];
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n < a.N) {
                    float v = acc[i][j];
                    if (a.epi == LIN_SOFTCAP) v = a.cap * tanhf(v / a.cap);
                    else if (a.epi == LIN_RELU2) { v = fmaxf(v, 0.f); v *= v; }
                    C[(size_t)r * a.ldc + n] = v;
                }
            }
        }
    }
}

// ------------------------------------------------------------------ linear: few rows (decode)
// A CTA of 8 warps owns 32 output columns (16 column pairs with the SwiGLU epilogue) of one problem and walks its rows
// LROWS at a time: a 512-wide slice of those rows is staged in shared memory once and reused by every column, each warp
// streams the weights of its columns 16 bytes per lane per load, so the weights are read once per LROWS rows.
constexpr int LROWS = 16, LKC = 512, LWARPS = 8;

template <bool PAIR, bool VEC>
__global__ void __launch_bounds__(LWARPS * 32) linear_rows_kernel(LinearArgs a) {
    constexpr int CPW = PAIR ? 2 : 4;                 // output columns per warp
    constexpr int WR = PAIR ? 2 * CPW : CPW;          // weight rows per warp
    __shared__ __align__(16) float sA[LROWS][LKC];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cols = PAIR ? a.N / 2 : a.N;
    const int p = blockIdx.y;
    const int col0 = (blockIdx.x * LWARPS + wid) * CPW;
    int r0 = 0, r1 = a.M;
    if (a.seg) { r0 = a.seg[p]; r1 = a.seg[p + 1]; }
    if (r1 <= r0) return;
    const float* A = a.A + (size_t)p * a.a_col_stride;
    const __nv_bfloat16* W = a.W + (size_t)p * a.w_stride;
    float* C = a.C + (size_t)p * a.c_col_stride;
    const __nv_bfloat16* wrow[WR];
    bool wok[WR];
#pragma unroll
    for (int c = 0; c < WR; ++c) {
        const int n = PAIR ? 2 * col0 + c : col0 + c;
        wok[c] = n < a.N;
        wrow[c] = W + (size_t)(wok[c] ? n : 0) * a.ldw;
    }
    for (int rb = r0; rb < r1; rb += LROWS) {
        const int nr = min(LROWS, r1 - rb);
        float acc[WR][LROWS];
#pragma unroll
        for (int c = 0; c < WR; ++c)
#pragma unroll
            for (int i = 0; i < LROWS; ++i) acc[c][i] = 0.f;
        for (int k0 = 0; k0 < a.K; k0 += LKC) {
            const int kc = min(LKC, a.K - k0);
            __syncthreads();
            for (int i = wid; i < nr; i += LWARPS) {          // a warp per row
                const int r = rb + i;
                const float* src = A + (size_t)(a.a_rows ? a.a_rows[r] : r) * a.lda + k0;
                if (VEC) {
                    for (int k = lane * 4; k < kc; k += 128)
                        *reinterpret_cast<float4*>(&sA[i][k]) = *reinterpret_cast<const float4*>(src + k);
                } else {
                    for (int k = lane; k < kc; k += 32) sA[i][k] = src[k];
                }
            }
            __syncthreads();
            if (VEC) {
                for (int k = lane * 8; k < kc; k += 256) {
                    float wv[WR][8];
#pragma unroll
                    for (int c = 0; c < WR; ++c) {
                        uint4 t = make_uint4(0u, 0u, 0u, 0u);
                        if (wok[c]) t = __ldg(reinterpret_cast<const uint4*>(wrow[c] + k0 + k));
                        wv[c][0] = bf16_lo(t.x); wv[c][1] = bf16_hi(t.x); wv[c][2] = bf16_lo(t.y); wv[c][3] = bf16_hi(t.y);
                        wv[c][4] = bf16_lo(t.z); wv[c][5] = bf16_hi(t.z); wv[c][6] = bf16_lo(t.w); wv[c][7] = bf16_hi(t.w);
                    }
#pragma unroll
                    for (int i = 0; i < LROWS; ++i) {
                        if (i < nr) {
                            const float4 x0 = *reinterpret_cast<const float4*>(&sA[i][k]);
                            const float4 x1 = *reinterpret_cast<const float4*>(&sA[i][k + 4]);
                            const float xa[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                            for (int c = 0; c < WR; ++c)
#pragma unroll
                                for (int e = 0; e < 8; ++e) acc[c][i] = fmaf(xa[e], wv[c][e], acc[c][i]);
                        }
                    }
                }
            } else {
                for (int k = lane; k < kc; k += 32) {
                    float wv[WR];
#pragma unroll
                    for (int c = 0; c < WR; ++c) wv[c] = wok[c] ? __bfloat162float(wrow[c][k0 + k]) : 0.f;
#pragma unroll
                    for (int i = 0; i < LROWS; ++i)
                        if (i < nr) {
                            const float x = sA[i][k];
#pragma unroll
                            for (int c = 0; c < WR; ++c) acc[c][i] = fmaf(x, wv[c], acc[c][i]);
                        }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
#pragma unroll
            for (int i = 0; i < LROWS; ++i) {
                if (i >= nr) continue;               // uniform over the warp
                float v;
                if (PAIR) {
                    const float g = warp_sum(acc[2 * c][i]), u = warp_sum(acc[2 * c + 1][i]);
                    v = g / (1.f + expf(-g)) * u;
                } else {
                    v = warp_sum(acc[c][i]);
                    if (a.epi == LIN_SOFTCAP) v = a.cap * tanhf(v / a.cap);
                    else if (a.epi == LIN_RELU2) { v = fmaxf(v, 0.f); v *= v; }
                }
                if (lane == 0 && col0 + c < cols) C[(size_t)(rb + i) * a.ldc + col0 + c] = v;
            }
        }
    }
}

int launch_linear(const LinearArgs& a, int rows_bound, cudaStream_t stream) {
    if (rows_bound <= 0 || a.N <= 0) return 0;
    FT_REQUIRE(a.K >= 1 && a.P >= 1, "linear: bad sizes");
    FT_REQUIRE(a.epi != LIN_SWIGLU_PAIR || (a.N & 1) == 0, "linear: the paired epilogue needs an even number of rows");
    // few rows per problem: one warp per output column, the weights stream once
    const bool few = a.seg ? rows_bound <= 4 * LROWS : rows_bound <= 2 * LROWS;
    if (few) {
        const bool pair = a.epi == LIN_SWIGLU_PAIR;
        const int cols = pair ? a.N / 2 : a.N;
        const int per_cta = LWARPS * (pair ? 2 : 4);
        const bool v8 = (a.K & 7) == 0 && (a.ldw & 7) == 0 && (a.lda & 3) == 0 && (a.a_col_stride & 3) == 0 &&
                        (a.w_stride & 7) == 0 && ((uintptr_t)a.A & 15) == 0 && ((uintptr_t)a.W & 15) == 0;
        dim3 grid((cols + per_cta - 1) / per_cta, a.P);
        if (pair) {
            if (v8) linear_rows_kernel<true, true><<<grid, LWARPS * 32, 0, stream>>>(a);
            else linear_rows_kernel<true, false><<<grid, LWARPS * 32, 0, stream>>>(a);
        } else {
            if (v8) linear_rows_kernel<false, true><<<grid, LWARPS * 32, 0, stream>>>(a);
            else linear_rows_kernel<false, false><<<grid, LWARPS * 32, 0, stream>>>(a);
        }
        FT_CHECK_CUDA(cudaGetLastError());
        return 0;
    }
    const bool vec = (a.lda & 3) == 0 && (a.ldw & 3) == 0 && (a.a_col_stride & 3) == 0 && (a.w_stride & 3) == 0 &&
                     ((uintptr_t)a.A & 15) == 0 && ((uintptr_t)a.W & 7) == 0;
    dim3 grid((a.N + LBN - 1) / LBN, 1, 1);
    if (a.seg) grid.y = (rows_bound + LBM - 1) / LBM + a.P;
    else { grid.y = (a.M + LBM - 1) / LBM; grid.z = a.P; }
    if (vec) linear_tile_kernel<true><<<grid, LTHREADS, 0, stream>>>(a);
    else linear_tile_kernel<false><<<grid, LTHREADS, 0, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ bf16 planes for the tensor-core projections
// v = hi + lo with hi = bf16(v), lo = bf16(v - hi): the tcgen05 GEMM multiplies both planes into one fp32 accumulator, which
// keeps about 16 mantissa bits of an fp32 activation.
__device__ __forceinline__ void store_planes(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t i, float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
}

__global__ void to_planes_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                 size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        store_planes(hi, lo, i, x[i]);
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

// planes of the rows an index list names: out row i = planes(src[idx[i]])
__global__ void gather_planes_kernel2(const float* __restrict__ src, const int* __restrict__ idx, __nv_bfloat16* __restrict__ hi,
                                      __nv_bfloat16* __restrict__ lo, int W) {
    const size_t i = blockIdx.x;
    const float* r = src + (size_t)idx[i] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) store_planes(hi, lo, i * W + c, r[c]);
}

// gu [rows][2 ff] with columns (2j, 2j+1) = (gate_j, up_j)  ->  planes of silu(gate) * up, [rows][ff]
__global__ void swiglu_planes_kernel(const float* __restrict__ gu, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                     size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float2 v = reinterpret_cast<const float2*>(gu)[i];
        store_planes(hi, lo, i, v.x / (1.f + expf(-v.x)) * v.y);
    }
}

// u [rows][ff]  ->  planes of relu(u)^2
__global__ void relu2_planes_kernel(const float* __restrict__ u, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                    size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(u[i], 0.f);
        store_planes(hi, lo, i, v * v);
    }
}

int launch_gather_planes_rows(const float* src, const int* idx, void* hi, void* lo, int n, int W, cudaStream_t stream) {
    gather_planes_kernel2<<<n, 256, 0, stream>>>(src, idx, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, W);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}
int launch_swiglu_planes(const float* gu, void* hi, void* lo, size_t n, cudaStream_t stream, int act) {
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
    if (act == FT_ACT_RELU2) relu2_planes_kernel<<<blocks, 256, 0, stream>>>(gu, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n);
    else swiglu_planes_kernel<<<blocks, 256, 0, stream>>>(gu, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int launch_to_planes(const float* x, void* hi, void* lo, size_t n, cudaStream_t stream) {
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
    to_planes_kernel<<<blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}
int launch_softcap(float* x, size_t n, float cap, cudaStream_t stream) {
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
    softcap_kernel<<<blocks, 256, 0, stream>>>(x, n, cap);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ embedding / residual update, fused with the next norm
// hn[t] = x[t] / sqrt(mean(x[t]^2) + eps) * gain, the gain being one number.
__global__ void __launch_bounds__(256)
embed_norm_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed, float* __restrict__ x,
                  float* __restrict__ hn, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo, int W, float eps,
                  float gain, const float* __restrict__ gain_w) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const __nv_bfloat16* e = embed + (size_t)tokens[t] * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = __bfloat162float(e[c]);
        x[(size_t)t * W + c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = gain / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = __bfloat162float(e[c]) * r;
        if (gain_w) v *= gain_w[c];
        hn[(size_t)t * W + c] = v;
        if (hi) store_planes(hi, lo, (size_t)t * W + c, v);
    }
}

// x[t] += sigmoid(rg1[t] + b1) * mix[t] + sigmoid(rg2[t] + b2) * sum_k wt[t, k] * eout[slot_pos[t, k]]   (feed-forward
// part only when top > 0), then the next norm of the row.  rg1 / rg2 are column ranges of the input projection `proj`.
__global__ void __launch_bounds__(256)
combine_norm_kernel(float* __restrict__ x, float* __restrict__ hn, const float* __restrict__ proj, int ldp, int o_rg1,
                    int o_rg2, const float* __restrict__ rg_bias, const float* __restrict__ mix,
                    const float* __restrict__ eout, const float* __restrict__ wt, const int* __restrict__ slot_pos,
                    int top, int W, float eps, float gain, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    __shared__ float red[33];
    extern __shared__ float row[];
    const int t = blockIdx.x;
    const float* pr = proj + (size_t)t * ldp;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float y = sigmoid_exact(pr[o_rg1 + c] + rg_bias[c]) * mix[(size_t)t * W + c];
        if (top > 0) {
            float f = 0.f;
            for (int k = 0; k < top; ++k)
                f = fmaf(wt[(size_t)t * top + k], eout[(size_t)slot_pos[(size_t)t * top + k] * W + c], f);
            y += sigmoid_exact(pr[o_rg2 + c] + rg_bias[W + c]) * f;
        }
        const float v = x[(size_t)t * W + c] + y;
        x[(size_t)t * W + c] = v;
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = gain / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = row[c] * r;
        hn[(size_t)t * W + c] = v;
        if (hi) store_planes(hi, lo, (size_t)t * W + c, v);
    }
}

// rows of the normed stream that the head reads: out[i] = hn[idx[i]]
__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ idx, float* __restrict__ dst, int W) {
    const int i = blockIdx.x;
    const float* s = src + (size_t)idx[i] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[(size_t)i * W + c] = s[c];
}

int launch_embed_norm(const int* tokens, const void* embed, float* x, float* hn, void* hi, void* lo, int T, int W, float eps,
                      float gain, const float* gain_w, cudaStream_t stream) {
    embed_norm_kernel<<<T, 256, 0, stream>>>(tokens, (const __nv_bfloat16*)embed, x, hn, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo,
                                             W, eps, gain_w ? 1.f : gain, gain_w);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}
int launch_combine_norm(float* x, float* hn, const float* proj, int ldp, int o_rg1, int o_rg2, const float* rg_bias,
                        const float* mix, const float* eout, const float* wt, const int* slot_pos, int top, int T, int W,
                        float eps, float gain, void* hi, void* lo, cudaStream_t stream) {
    combine_norm_kernel<<<T, 256, (size_t)W * 4, stream>>>(x, hn, proj, ldp, o_rg1, o_rg2, rg_bias, mix, eout, wt, slot_pos,
                                                          top, W, eps, gain, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}
int launch_gather_rows(const float* src, const int* idx, float* dst, int n, int W, cudaStream_t stream) {
    gather_rows_kernel<<<n, 256, 0, stream>>>(src, idx, dst, W);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ latent attention
// The latent of token t: c = raw / sqrt(mean(raw^2) + eps) * w, written to page_table[seq_rows[t]][pos / 64], row pos % 64
// of the layer's cache [page][64][rank] fp32.
__global__ void __launch_bounds__(128)
latent_write_kernel(const float* __restrict__ proj, int ldp, int o_dkv, const float* __restrict__ w, float* __restrict__ cache,
                    __nv_bfloat16* __restrict__ cache16, const int* __restrict__ positions, const int* __restrict__ seq_rows, const int* __restrict__ page_table,
                    int max_pages, int rank, float eps) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const float* raw = proj + (size_t)t * ldp + o_dkv;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) ss += raw[c] * raw[c];
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)rank + eps);
    const int pos = positions[t];
    const int page = page_table[(size_t)seq_rows[t] * max_pages + pos / kKvTile];
    const size_t at = ((size_t)page * kKvTile + pos % kKvTile) * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = raw[c] * r * w[c];
        cache[at + c] = v;
        if (cache16) cache16[at + c] = __float2bfloat16_rn(v);      // the tensor-core attention's copy
    }
}

// One warp per (token, head, key range): the query in latent space stays in registers (NR values per lane), keys = values =
// the cached latents, online softmax in fp32.  Keys are taken KB at a time: their rows are all requested before the first
// is used and the KB score reductions interleave, so the loop waits for memory once per block instead of once per key.
// With n_split == 1 the warp finishes its (token, head): divides by the softmax sum and scales by the head's output gate
// sigmoid(gate logit) — the value expansion that follows is linear, so gating before it is the same.  With n_split > 1
// (few tokens: decode) it covers the s-th share of the keys and leaves (max, sum, unnormalised result) for the merge.
template <int NR, int KB>
__global__ void __launch_bounds__(128)
latent_attn_kernel(const float* __restrict__ qlat, const float* __restrict__ cache, const float* __restrict__ proj, int ldp,
                   int o_gate, float* __restrict__ out, float* __restrict__ part, const int* __restrict__ positions,
                   const int* __restrict__ seq_rows, const int* __restrict__ page_table, int max_pages, int H, int rank,
                   float scale, int n_pairs, int n_split) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int split = blockIdx.y;
    if (pair >= n_pairs) return;
    const int t = pair / H, h = pair % H;
    const float* q = qlat + ((size_t)t * H + h) * rank;
    float qr[NR], acc[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int c = lane + 32 * i;
        qr[i] = c < rank ? q[c] * scale : 0.f;
        acc[i] = 0.f;
    }
    const int n_keys = positions[t] + 1;
    int j_lo = 0, j_hi = n_keys;
    if (n_split > 1) {          // shares of whole pages
        const int share = ((n_keys + n_split - 1) / n_split + kKvTile - 1) / kKvTile * kKvTile;
        j_lo = min(split * share, n_keys);
        j_hi = min(j_lo + share, n_keys);
    }
    const int* pt = page_table + (size_t)seq_rows[t] * max_pages;
    float m = -INFINITY, l = 0.f;
    for (int j0 = j_lo; j0 < j_hi; j0 += KB) {
        float cv[KB][NR], sc[KB];
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const int j = min(j0 + b, j_hi - 1);
            const float* c = cache + ((size_t)pt[j / kKvTile] * kKvTile + j % kKvTile) * rank;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int cc = lane + 32 * i;
                cv[b][i] = cc < rank ? c[cc] : 0.f;
            }
        }
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            float x = 0.f;
#pragma unroll
            for (int i = 0; i < NR; ++i) x = fmaf(qr[i], cv[b][i], x);
            sc[b] = x;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int b = 0; b < KB; ++b) sc[b] += __shfl_xor_sync(0xffffffffu, sc[b], o);
        float mn = m;
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            if (j0 + b >= j_hi) sc[b] = -INFINITY;
            mn = fmaxf(mn, sc[b]);
        }
        const float corr = expf(m - mn);
        l *= corr;
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[i] *= corr;
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const float pw = expf(sc[b] - mn);          // 0 for the padding of the last block
            l += pw;
#pragma unroll
            for (int i = 0; i < NR; ++i) acc[i] = fmaf(pw, cv[b][i], acc[i]);
        }
        m = mn;
    }
    if (n_split > 1) {
        float* p = part + ((size_t)pair * n_split + split) * (rank + 2);
        if (lane == 0) { p[0] = m; p[1] = l; }
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int c = lane + 32 * i;
            if (c < rank) p[2 + c] = acc[i];
        }
        return;
    }
    const float g = sigmoid_exact(proj[(size_t)t * ldp + o_gate + h]) / l;
    float* o = out + ((size_t)t * H + h) * rank;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) o[c] = acc[i] * g;
    }
}

// The shares of one (token, head) put together: one warp each.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part, const float* __restrict__ proj, int ldp, int o_gate, float* __restrict__ out,
                    int H, int rank, int n_pairs, int n_split) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const float* p = part + (size_t)pair * n_split * (rank + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_split; ++s) m = fmaxf(m, p[(size_t)s * (rank + 2)]);
    float l = 0.f;
    for (int s = 0; s < n_split; ++s) {
        const float ms = p[(size_t)s * (rank + 2)];
        if (ms > -INFINITY) l += p[(size_t)s * (rank + 2) + 1] * expf(ms - m);
    }
    const int t = pair / H, h = pair % H;
    const float g = sigmoid_exact(proj[(size_t)t * ldp + o_gate + h]) / l;
    for (int c = lane; c < rank; c += 32) {
        float a = 0.f;
        for (int s = 0; s < n_split; ++s) {
            const float ms = p[(size_t)s * (rank + 2)];
            if (ms > -INFINITY) a = fmaf(p[(size_t)s * (rank + 2) + 2 + c], expf(ms - m), a);
        }
        out[(size_t)pair * rank + c] = a * g;
    }
}

int launch_latent_write(const float* proj, int ldp, int o_dkv, const float* w, float* cache, void* cache16, const int* positions,
                        const int* seq_rows, const int* page_table, int max_pages, int rank, float eps, int T,
                        cudaStream_t stream) {
    latent_write_kernel<<<T, 128, 0, stream>>>(proj, ldp, o_dkv, w, cache, (__nv_bfloat16*)cache16, positions, seq_rows, page_table,
                                               max_pages, rank, eps);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// The serving form of the same attention on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulation and
// softmax): one CTA per (token, key share, group of 16 heads).  The 16 heads are the M rows of every product, so all rows
// of a tile see the same keys and one mask.  Each of the four warps takes every fourth 16-key tile of the share: the tile
// (16 latents from the bf16 copy of the cache) is copied into the warp's own double buffer with cp.async one tile ahead,
// S = Q C^T (ldmatrix fragments of Q and of the tile), online softmax in registers, O += P C with the SAME tile read
// through ldmatrix.trans — keys and values are one array.  The warps' (max, sum, O) are merged through shared memory.
// rank = 32 * RK <= 256 (O is rank / 8 accumulator tiles per thread).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <int RK>
__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(const float* __restrict__ qlat, const __nv_bfloat16* __restrict__ cache16, const float* __restrict__ proj,
                       int ldp, int o_gate, float* __restrict__ out, float* __restrict__ part, const int* __restrict__ positions,
                       const int* __restrict__ seq_rows, const int* __restrict__ page_table, int max_pages, int H, float scale,
                       int n_split) {
    constexpr int RANK = 32 * RK, RS = RANK * 2 + 16;      // row stride in bytes: 16 bytes of padding keep ldmatrix conflict-free
    constexpr int TILE = 16 * RS;
    extern __shared__ __align__(16) uint8_t lat_smem[];
    uint8_t* Qs = lat_smem;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* kbuf = lat_smem + TILE + (size_t)warp * 2 * TILE;
    const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * 16;
    for (int idx = threadIdx.x; idx < 16 * RANK; idx += 128) {
        const int r = idx / RANK, c = idx % RANK;
        const float v = h0 + r < H ? qlat[((size_t)t * H + h0 + r) * RANK + c] * scale : 0.f;
        *reinterpret_cast<__nv_bfloat16*>(Qs + r * RS + c * 2) = __float2bfloat16_rn(v);
    }
    __syncthreads();
    const int n_keys = positions[t] + 1;
    int j_lo = 0, j_hi = n_keys;
    if (n_split > 1) {
        const int share = ((n_keys + n_split - 1) / n_split + kKvTile - 1) / kKvTile * kKvTile;
        j_lo = min(split * share, n_keys);
        j_hi = min(j_lo + share, n_keys);
    }
    const int* pt = page_table + (size_t)seq_rows[t] * max_pages;
    const int n_tiles = (j_hi - j_lo + 15) / 16;
    auto stage = [&](int tile, int buf) {
        const int key0 = j_lo + tile * 16;
        uint8_t* dst = kbuf + buf * TILE;
        for (int i = lane; i < 16 * 4 * RK; i += 32) {          // 16 rows of 4 * RK 16-byte pieces
            const int r = i / (4 * RK), ch = i % (4 * RK);
            const int j = min(key0 + r, j_hi - 1);
            cp_async16(dst + r * RS + ch * 16, cache16 + ((size_t)pt[j / kKvTile] * kKvTile + j % kKvTile) * RANK + ch * 8);
        }
        cp_async_commit();
    };
    float o[4 * RK][4];
#pragma unroll
    for (int nt = 0; nt < 4 * RK; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;      // rows g and g + 8
    const int g = lane >> 2, tq = lane & 3;
    const uint32_t q_addr = smem_u32(Qs) + ((lane & 7) + ((lane >> 3) & 1) * 8) * RS + (lane >> 4) * 16;
    if (warp < n_tiles) stage(warp, 0);
    for (int tile = warp, it = 0; tile < n_tiles; tile += 4, ++it) {
        const int cur = it & 1;
        if (tile + 4 < n_tiles) { stage(tile + 4, cur ^ 1); cp_async_wait_1(); }
        else cp_async_wait_all();
        __syncwarp();
        const uint32_t kb = smem_u32(kbuf + cur * TILE);
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int kp = 0; kp < RK; ++kp) {                        // 32 latent channels per round
            uint32_t a0[4], a1[4];
            ldmatrix_x4(q_addr + (kp * 4) * 16, a0[0], a0[1], a0[2], a0[3]);
            ldmatrix_x4(q_addr + (kp * 4 + 2) * 16, a1[0], a1[1], a1[2], a1[3]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + (8 * j + (lane & 7)) * RS + (kp * 4 + (lane >> 3)) * 16, b0, b1, b2, b3);
                mma_bf16_16816(sc[j], a0[0], a0[1], a0[2], a0[3], b0, b1);
                mma_bf16_16816(sc[j], a1[0], a1[1], a1[2], a1[3], b2, b3);
            }
        }
        const int key0 = j_lo + tile * 16 + 2 * tq;
        float ta = -INFINITY, tb = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (key0 + 8 * j + e >= j_hi) sc[j][e] = sc[j][2 + e] = -INFINITY;
                ta = fmaxf(ta, sc[j][e]);
                tb = fmaxf(tb, sc[j][2 + e]);
            }
        ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 1));
        ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 2));
        tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 1));
        tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 2));
        const float na = fmaxf(m_a, ta), nb = fmaxf(m_b, tb);      // finite: the tile's first key is never masked
        const float alpha_a = expf(m_a - na), alpha_b = expf(m_b - nb);
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sc[j][e] = expf(sc[j][e] - na);
                sc[j][2 + e] = expf(sc[j][2 + e] - nb);
                sa += sc[j][e];
                sb += sc[j][2 + e];
            }
        l_a = l_a * alpha_a + sa;
        l_b = l_b * alpha_b + sb;
        m_a = na;
        m_b = nb;
        const uint32_t pa0 = pack_bf16(sc[0][0], sc[0][1]), pa1 = pack_bf16(sc[0][2], sc[0][3]);
        const uint32_t pa2 = pack_bf16(sc[1][0], sc[1][1]), pa3 = pack_bf16(sc[1][2], sc[1][3]);
        const int vrow = ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
        for (int np = 0; np < 2 * RK; ++np) {                    // 16 latent channels per round
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(kb + vrow * RS + (2 * np + (lane >> 4)) * 16, b0, b1, b2, b3);
            o[2 * np][0] *= alpha_a; o[2 * np][1] *= alpha_a; o[2 * np][2] *= alpha_b; o[2 * np][3] *= alpha_b;
            o[2 * np + 1][0] *= alpha_a; o[2 * np + 1][1] *= alpha_a; o[2 * np + 1][2] *= alpha_b; o[2 * np + 1][3] *= alpha_b;
            mma_bf16_16816(o[2 * np], pa0, pa1, pa2, pa3, b0, b1);
            mma_bf16_16816(o[2 * np + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
        __syncwarp();
    }
    // the warp's record in its own (now idle) buffer: 16 rows of rank results, then max and sum
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    constexpr int REC = RANK + 2;
    float* rec = reinterpret_cast<float*>(kbuf);
#pragma unroll
    for (int nt = 0; nt < 4 * RK; ++nt) {
        rec[g * REC + nt * 8 + 2 * tq] = o[nt][0];
        rec[g * REC + nt * 8 + 2 * tq + 1] = o[nt][1];
        rec[(g + 8) * REC + nt * 8 + 2 * tq] = o[nt][2];
        rec[(g + 8) * REC + nt * 8 + 2 * tq + 1] = o[nt][3];
    }
    if (tq == 0) {
        rec[g * REC + RANK] = m_a; rec[g * REC + RANK + 1] = l_a;
        rec[(g + 8) * REC + RANK] = m_b; rec[(g + 8) * REC + RANK + 1] = l_b;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * RANK; idx += 128) {
        const int r = idx / RANK, c = idx % RANK;
        if (h0 + r >= H) continue;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, reinterpret_cast<const float*>(lat_smem + TILE + (size_t)w * 2 * TILE)[r * REC + RANK]);
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* rw = reinterpret_cast<const float*>(lat_smem + TILE + (size_t)w * 2 * TILE) + r * REC;
            if (rw[RANK] > -INFINITY) {
                const float f = expf(rw[RANK] - m);
                l = fmaf(rw[RANK + 1], f, l);
                a = fmaf(rw[c], f, a);
            }
        }
        const size_t pair = (size_t)t * H + h0 + r;
        if (n_split > 1) {
            float* p = part + (pair * n_split + split) * REC;
            p[2 + c] = a;
            if (c == 0) { p[0] = m; p[1] = l; }
        } else {
            out[pair * RANK + c] = a / l * sigmoid_exact(proj[(size_t)t * ldp + o_gate + h0 + r]);
        }
    }
}

int latent_attn_splits(int T, int H) {
    const int pairs = T * H;
    if (pairs >= kLatentSplitPairs) return 1;
    return std::max(1, std::min(kLatentMaxSplits, kLatentSplitPairs / std::max(pairs, 1)));
}

bool latent_attn_mma_ok(int rank) { return rank % 32 == 0 && rank >= 32 && rank <= 256; }

int launch_latent_attn(const float* qlat, const float* cache, const void* cache16, const float* proj, int ldp, int o_gate,
                       float* out, float* part, const int* positions, const int* seq_rows, const int* page_table, int max_pages,
                       int H, int rank, float scale, int T, cudaStream_t stream) {
    const int n_pairs = T * H;
    const int n_split = part ? latent_attn_splits(T, H) : 1;
    if (cache16 && latent_attn_mma_ok(rank)) {
        const dim3 grid(T, n_split, (H + 15) / 16);
        const size_t smem = (size_t)9 * 16 * (rank * 2 + 16);
#define FT_LATM(RK_)                                                                                                        \
    case RK_: {                                                                                                             \
        static PerDeviceFlag attr;                                                                                          \
        if (!attr.done()) {                                                                                                 \
            FT_CHECK_CUDA(cudaFuncSetAttribute(latent_attn_mma_kernel<RK_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                               9 * 16 * (RK_ * 64 + 16)));                                                  \
            attr.mark();                                                                                                    \
        }                                                                                                                   \
        latent_attn_mma_kernel<RK_><<<grid, 128, smem, stream>>>(qlat, (const __nv_bfloat16*)cache16, proj, ldp, o_gate, out, \
                                                                 part, positions, seq_rows, page_table, max_pages, H, scale, \
                                                                 n_split);                                                  \
        break;                                                                                                              \
    }
        switch (rank / 32) {
            FT_LATM(1) FT_LATM(2) FT_LATM(3) FT_LATM(4) FT_LATM(5) FT_LATM(6) FT_LATM(7) FT_LATM(8)
            default: break;
        }
#undef FT_LATM
        FT_CHECK_CUDA(cudaGetLastError());
        if (n_split > 1) {
            latent_merge_kernel<<<(n_pairs + 3) / 4, 128, 0, stream>>>(part, proj, ldp, o_gate, out, H, rank, n_pairs, n_split);
            FT_CHECK_CUDA(cudaGetLastError());
        }
        return 0;
    }
    const dim3 grid((n_pairs + 3) / 4, n_split);
#define FT_LAT(NR_, KB_)                                                                                                   \
    latent_attn_kernel<NR_, KB_><<<grid, 128, 0, stream>>>(qlat, cache, proj, ldp, o_gate, out, part, positions, seq_rows, \
                                                           page_table, max_pages, H, rank, scale, n_pairs, n_split)
    if (rank <= 32) FT_LAT(1, 8);
    else if (rank <= 64) FT_LAT(2, 8);
    else if (rank <= 128) FT_LAT(4, 8);
    else if (rank <= 256) FT_LAT(8, 4);
    else if (rank <= 512) FT_LAT(16, 4);
    else { FT_REQUIRE(rank <= 1024, "latent attention: latent size %d is beyond 1024", rank); FT_LAT(32, 2); }
#undef FT_LAT
    FT_CHECK_CUDA(cudaGetLastError());
    if (n_split > 1) {
        latent_merge_kernel<<<(n_pairs + 3) / 4, 128, 0, stream>>>(part, proj, ldp, o_gate, out, H, rank, n_pairs, n_split);
        FT_CHECK_CUDA(cudaGetLastError());
    }
    return 0;
}

// ------------------------------------------------------------------ channel delta
// Per token: the three short convolutions over time + SiLU (inputs before the step's first token come from the session's
// tail of raw inputs; zeros before position 0), unit norms of q and k per head (q also times dim^-1/2), the decay
// exp(-exp(A_log_h) * softplus(a + dt_bias)) per head and key channel, beta = sigmoid.
// qkv out: [T][channels] with channels = 2 * kvh * dim + heads * vdim in the order q | k | v.
__global__ void __launch_bounds__(256)
delta_prep_kernel(DeltaArgs a) {
    extern __shared__ float sh[];
    const int t = blockIdx.x;
    const int req = a.seq_rows[t];
    const int r = t - a.req_start[req];              // index inside this step's portion
    const int pos0 = a.req_pos0[req];
    const int qk = a.kvh * a.dim, ch = 2 * qk + a.heads * a.vdim;
    const float* tail = a.state + (size_t)a.req_slot[req] * a.slot_stride + a.tail_off;
    const int taps = a.taps;
    for (int c = threadIdx.x; c < ch; c += blockDim.x) {
        float s = 0.f;
        for (int i = 0; i < taps; ++i) {
            const int back = taps - 1 - i;
            float v;
            if (r - back >= 0) v = a.proj[(size_t)(t - back) * a.ldp + a.o_q + c];
            else if (pos0 + r - back >= 0) v = tail[(size_t)c * (taps - 1) + (taps - 1 + r - back)];
            else v = 0.f;
            s = fmaf(a.conv[(size_t)c * taps + i], v, s);
        }
        sh[c] = s / (1.f + expf(-s));
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* dst = a.qkv + (size_t)t * ch;
    for (int hh = wid; hh < 2 * a.kvh; hh += nw) {          // q heads, then k heads
        const float* v = sh + (size_t)hh * a.dim;
        float ss = 0.f;
        for (int d = lane; d < a.dim; d += 32) ss += v[d] * v[d];
        ss = warp_sum(ss);
        float sc = 1.f / sqrtf(ss + 1e-6f);
        if (hh < a.kvh) sc *= 1.f / sqrtf((float)a.dim);
        for (int d = lane; d < a.dim; d += 32) dst[(size_t)hh * a.dim + d] = v[d] * sc;
    }
    for (int c = 2 * qk + threadIdx.x; c < ch; c += blockDim.x) dst[c] = sh[c];
    const int hd = a.heads * a.dim;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        // one decay per head and key channel, or (head_decay) one per head, written to all of the head's channels
        const float z = a.head_decay ? a.araw[(size_t)t * a.ld_araw + i / a.dim] + a.dt_bias[i / a.dim]
                                     : a.araw[(size_t)t * hd + i] + a.dt_bias[i];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        a.decay[(size_t)t * hd + i] = expf(-expf(a.a_log[i / a.dim]) * sp);
    }
    for (int h = threadIdx.x; h < a.heads; h += blockDim.x)
        a.beta[(size_t)t * a.heads + h] = sigmoid_exact(a.proj[(size_t)t * a.ldp + a.o_beta + h]);
}

// New tail of raw convolution inputs per (request, channel): the last taps-1 entries of (old tail ++ this step's inputs).
__global__ void delta_tail_kernel(DeltaArgs a, int n_req) {
    const int req = blockIdx.y;
    const int ch = 2 * a.kvh * a.dim + a.heads * a.vdim;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= ch || req >= n_req) return;
    const int n = a.req_start[req + 1] - a.req_start[req], pos0 = a.req_pos0[req], keep = a.taps - 1;
    float* tail = a.state + (size_t)a.req_slot[req] * a.slot_stride + a.tail_off + (size_t)c * keep;
    float v[16];
    for (int i = 0; i < keep; ++i) {
        const int src = n + i;                      // index into old tail (keep entries) ++ inputs (n entries)
        if (src < keep) v[i] = pos0 > 0 ? tail[src] : 0.f;
        else v[i] = a.proj[(size_t)(a.req_start[req] + src - keep) * a.ldp + a.o_q + c];
    }
    for (int i = 0; i < keep; ++i) tail[i] = v[i];
}

// The recurrence, one CTA per (request, head, block of DCOLS state columns).  Per token
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// is local to a column of the state S [dim][vdim].  Four neighbouring lanes share a column, each holding a run of DPT key
// channels of it in registers, so the two sums over key channels are two short chains plus two shuffles.
// q, k, g, v, beta of DCHUNK tokens at a time are copied into shared memory asynchronously (cp.async), one chunk ahead
// of the one being computed.
constexpr int DCHUNK = 8, DCOLS = 32;

// Shared-memory layout of one staged token: q, k, g each as four runs of DPT channels (one per lane of a column's quad)
// with four floats of padding between runs, so that the quad's 16-byte reads fall into different banks; then v, then beta.
template <int DPT>
__host__ __device__ constexpr int delta_run() { return DPT + 4; }
__host__ __device__ inline int delta_token_floats(int dpt, int vdim) { return (12 * (dpt + 4) + vdim + 1 + 3) & ~3; }

// FULL: dim == 4 * DPT, every channel test is true at compile time (the tests otherwise compile to branches in the token loop).
template <int DPT, int MAXT, bool FULL>
__global__ void __launch_bounds__(MAXT)
delta_rule_kernel(DeltaArgs a) {
    extern __shared__ __align__(16) float sh[];
    constexpr int RUN = delta_run<DPT>();
    const int req = blockIdx.x, h = blockIdx.y;
    const int j = blockIdx.z * DCOLS + (threadIdx.x >> 2), part = threadIdx.x & 3;      // column, and which run of key channels
    const int kh = h / (a.heads / a.kvh);
    const int row0 = a.req_start[req], n = a.req_start[req + 1] - row0;
    const int dim = a.dim, vdim = a.vdim;
    const int qk = a.kvh * dim, ch = 2 * qk + a.heads * vdim, hd = a.heads * dim;
    float* S = a.state + (size_t)a.req_slot[req] * a.slot_stride + a.s_off + (size_t)h * dim * vdim;
    const bool live = j < vdim;
    const bool fresh = a.req_pos0[req] == 0;
    const int d0 = part * DPT;                    // this lane's channels: d0 .. d0 + DPT - 1
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) s[i] = (live && !fresh && d0 + i < dim) ? S[(size_t)(d0 + i) * vdim + j] : 0.f;
    const int per = delta_token_floats(DPT, vdim);
    const int o_k = 4 * RUN, o_g = 8 * RUN, o_v = 12 * RUN;
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    auto stage = [&](int c0, float* buf) {
        const int nc = min(DCHUNK, n - c0);
        for (int tt = wid; tt < nc; tt += nw) {          // a warp per token
            const size_t t = row0 + c0 + tt;
            float* dst = buf + (size_t)tt * per;
            const float* q = a.qkv + t * ch + (size_t)kh * dim;
            const float* g = a.decay + t * hd + (size_t)h * dim;
            const float* v = a.qkv + t * ch + 2 * qk + (size_t)h * vdim;
            for (int e = lane; e < dim; e += 32) {
                const int at = (e / DPT) * RUN + e % DPT;
                cp_async4(dst + at, q + e);
                cp_async4(dst + o_k + at, q + qk + e);
                cp_async4(dst + o_g + at, g + e);
            }
            for (int e = lane; e < vdim; e += 32) cp_async4(dst + o_v + e, v + e);
            if (lane == 0) cp_async4(dst + o_v + vdim, a.beta + t * a.heads + h);
        }
        cp_async_commit();
    };
    float* buf0 = sh;
    float* buf1 = sh + (size_t)DCHUNK * per;
    stage(0, buf0);
    for (int c0 = 0, it = 0; c0 < n; c0 += DCHUNK, ++it) {
        float* cur = (it & 1) ? buf1 : buf0;
        cp_async_wait_all();
        __syncthreads();                                  // chunk `it` has landed; everyone is done with the other buffer
        if (c0 + DCHUNK < n) stage(c0 + DCHUNK, (it & 1) ? buf0 : buf1);
        const int nc = min(DCHUNK, n - c0);
        for (int tt = 0; tt < nc; ++tt) {
            const float* base = cur + (size_t)tt * per;
            const float4* q4 = reinterpret_cast<const float4*>(base + part * RUN);
            const float4* k4 = reinterpret_cast<const float4*>(base + o_k + part * RUN);
            const float4* g4 = reinterpret_cast<const float4*>(base + o_g + part * RUN);
            float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                if (FULL || d0 + i < dim) {
                    const float4 gg = g4[i >> 2], kk = k4[i >> 2];
                    const float ga[4] = {gg.x, gg.y, gg.z, gg.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (FULL || d0 + i + e < dim) {
                            s[i + e] *= ga[e];
                            if (e & 1) dot1 = fmaf(s[i + e], ka[e], dot1);
                            else dot0 = fmaf(s[i + e], ka[e], dot0);
                        }
                }
            }
            float dot = dot0 + dot1;
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            const float u = live ? base[o_v + vdim] * (base[o_v + j] - dot) : 0.f;
            float oa = 0.f, ob = 0.f;
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                if (FULL || d0 + i < dim) {
                    const float4 kk = k4[i >> 2], qq = q4[i >> 2];
                    const float ka[4] = {kk.x, kk.y, kk.z, kk.w}, qa[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (FULL || d0 + i + e < dim) {
                            s[i + e] = fmaf(ka[e], u, s[i + e]);
                            if (e & 1) ob = fmaf(s[i + e], qa[e], ob);
                            else oa = fmaf(s[i + e], qa[e], oa);
                        }
                }
            }
            float o = oa + ob;
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (live && part == 0) a.o[(size_t)(row0 + c0 + tt) * ((size_t)a.heads * vdim) + (size_t)h * vdim + j] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (d0 + i < dim) S[(size_t)(d0 + i) * vdim + j] = s[i];
    }
}

// o[t, h, :] <- o / sqrt(mean(o^2) + eps) * w * act(gate[t, h, :]), one warp per (token, head); act = sigmoid or silu;
// gate rows have stride ldg
__global__ void __launch_bounds__(128)
delta_out_kernel(float* __restrict__ o, const float* __restrict__ gate, const float* __restrict__ w, int vdim, float eps,
                 int n_pairs, int heads, int ldg, int gate_act) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    float* p = o + (size_t)pair * vdim;
    const float* g = gate + (size_t)(pair / heads) * ldg + (size_t)(pair % heads) * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss += p[c] * p[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) p[c] = p[c] * r * w[c] * sigmoid_exact(g[c]) * (gate_act == 1 ? g[c] : 1.f);
}

int launch_delta(const DeltaArgs& a, const float* gate, const float* out_norm, float eps, int T, int n_req,
                 cudaStream_t stream, int ldg, int gate_act) {
    const int ch = 2 * a.kvh * a.dim + a.heads * a.vdim;
    FT_REQUIRE(a.taps >= 1 && a.taps <= 17, "channel delta: %d convolution taps are beyond 17", a.taps);
    FT_REQUIRE(a.dim <= 256 && a.vdim <= 256, "channel delta: head sizes %d / %d are beyond 256", a.dim, a.vdim);
    FT_REQUIRE((size_t)ch * 4 <= 200 * 1024, "channel delta: %d channels do not fit in shared memory", ch);
    static PerDeviceFlag attr;
    if (!attr.done()) {
        FT_CHECK_CUDA(cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr.mark();
    }
    delta_prep_kernel<<<T, 256, (size_t)ch * 4, stream>>>(a);
    FT_CHECK_CUDA(cudaGetLastError());
    if (a.taps > 1) {
        delta_tail_kernel<<<dim3((ch + 127) / 128, n_req), 128, 0, stream>>>(a, n_req);
        FT_CHECK_CUDA(cudaGetLastError());
    }
    const int threads = (4 * std::min(a.vdim, DCOLS) + 31) / 32 * 32;      // four lanes per state column, whole warps
    const int dpt = a.dim <= 32 ? 8 : a.dim <= 64 ? 16 : a.dim <= 128 ? 32 : 64;
    const size_t smem = (size_t)2 * DCHUNK * delta_token_floats(dpt, a.vdim) * 4;
    const dim3 grid(n_req, a.heads, (a.vdim + DCOLS - 1) / DCOLS);
#define FT_DELTA_ONE(DPT_, FULL_)                                                                           \
    do {                                                                                                    \
        if (smem > 48 * 1024)                                                                               \
            FT_CHECK_CUDA(cudaFuncSetAttribute(delta_rule_kernel<DPT_, 4 * DCOLS, FULL_>,                   \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
        delta_rule_kernel<DPT_, 4 * DCOLS, FULL_><<<grid, threads, smem, stream>>>(a);                      \
    } while (0)
#define FT_DELTA(DPT_)                                  \
    do {                                                \
        if (a.dim == 4 * DPT_) FT_DELTA_ONE(DPT_, true); \
        else FT_DELTA_ONE(DPT_, false);                 \
    } while (0)
    if (a.dim <= 32) FT_DELTA(8);
    else if (a.dim <= 64) FT_DELTA(16);
    else if (a.dim <= 128) FT_DELTA(32);
    else FT_DELTA(64);
#undef FT_DELTA
#undef FT_DELTA_ONE
    FT_CHECK_CUDA(cudaGetLastError());
    const int n_pairs = T * a.heads;
    delta_out_kernel<<<(n_pairs + 3) / 4, 128, 0, stream>>>(a.o, gate, out_norm, a.vdim, eps, n_pairs, a.heads,
                                                            ldg > 0 ? ldg : a.heads * a.vdim, gate_act);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ router
// One warp per token: s = softmax(z) over all E experts (or sigmoid(z) of each); a group's score is its largest s; only
// experts of the `keep` best groups can be chosen; the `top` largest s among them, lowest index first on a tie; weights = s
// as it is, or (normalise) divided by the sum of the chosen ones (+ 1e-20); then times `scale`.
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ proj, int ldp, int o_router, int E, int top, int groups, int keep, int* __restrict__ ids,
             float* __restrict__ wts, int T, int sigmoid_scores, int normalise, float scale) {
    extern __shared__ float sh[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + wid;
    if (t >= T) return;
    float* s = sh + (size_t)wid * (E + groups);     // scores, then group scores; a taken entry is set to -1
    float* gs = s + E;
    const float* z = proj + (size_t)t * ldp + o_router;
    if (sigmoid_scores) {
        for (int e = lane; e < E; e += 32) s[e] = sigmoid_exact(z[e]);
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - m); s[e] = v; sum += v; }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
    }
    __syncwarp();
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
        float b = -1.f;
        for (int i = 0; i < per; ++i) b = fmaxf(b, s[g * per + i]);
        gs[g] = b;
    }
    __syncwarp();
    // drop the groups that are not among the best `keep`: groups - keep rounds of "remove the smallest" would favour the
    // wrong side of ties, so pick the best `keep` and mark them by negating (score + 2)
    for (int r = 0; r < keep; ++r) {
        float bv = -1.f; int bi = 0x7fffffff;
        for (int g = lane; g < groups; g += 32) if (gs[g] >= 0.f && (gs[g] > bv)) { bv = gs[g]; bi = g; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0 && bi < groups) gs[bi] = -(bv + 2.f);
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        float bv = -1.f; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] < -1.f && s[e] >= 0.f && s[e] > bv) { bv = s[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            const int e = bi < E ? bi : 0;
            ids[(size_t)t * top + r] = e;
            wts[(size_t)t * top + r] = bi < E ? bv : 0.f;
            if (bi < E) s[bi] = -1.f;
        }
        __syncwarp();
    }
    if (lane == 0 && (normalise || scale != 1.f)) {
        float* w = wts + (size_t)t * top;
        float total = 0.f;
        for (int r = 0; r < top; ++r) total += w[r];
        for (int r = 0; r < top; ++r) w[r] = (normalise ? w[r] / (total + 1e-20f) : w[r]) * scale;
    }
}

// Counting sort of the T * top (token, choice) pairs by expert, one CTA: seg[e] .. seg[e+1] are the sorted places of
// expert e, slot_token[place] the token whose row the expert reads, slot_pos[pair] the place of a pair.  Within an expert the
// order is (token, choice) order, so the layout is the same from run to run.
__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ ids, int n_pairs, int top, int E, int* __restrict__ seg, int* __restrict__ slot_token,
                  int* __restrict__ slot_pos) {
    extern __shared__ int shi[];
    int* cnt = shi;                    // [E + 1]
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[ids[i] + 1], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int e = 0; e < E; ++e) cnt[e + 1] += cnt[e];
        for (int e = 0; e <= E; ++e) seg[e] = cnt[e];
    }
    __syncthreads();
    // stable placement: a warp per expert walks the pairs in order (ballot + prefix count)
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = wid; e < E; e += nw) {
        int base = cnt[e];
        for (int i0 = 0; i0 < n_pairs; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < n_pairs && ids[i] == e;
            const unsigned b = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int place = base + __popc(b & ((1u << lane) - 1u));
                slot_token[place] = i / top;
                slot_pos[i] = place;
            }
            base += __popc(b);
        }
    }
}

int launch_route(const float* proj, int ldp, int o_router, int E, int top, int groups, int keep, int* ids, float* wts,
                 int* seg, int* slot_token, int* slot_pos, int T, cudaStream_t stream, int route_kind, int normalise,
                 float scale) {
    FT_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && top >= 1 && top <= (E / groups) * keep,
               "router: %d experts, %d groups, keep %d, top %d do not fit together", E, groups, keep, top);
    const size_t smem = (size_t)4 * (E + groups) * 4;
    FT_REQUIRE(smem <= 48 * 1024 && (size_t)(E + 1) * 4 <= 48 * 1024, "router: %d experts are too many", E);
    route_kernel<<<(T + 3) / 4, 128, smem, stream>>>(proj, ldp, o_router, E, top, groups, keep, ids, wts, T,
                                                     route_kind == FT_ROUTE_SIGMOID, normalise, scale > 0.f ? scale : 1.f);
    FT_CHECK_CUDA(cudaGetLastError());
    route_sort_kernel<<<1, 1024, (size_t)(E + 1) * 4, stream>>>(ids, T * top, top, E, seg, slot_token, slot_pos);
    FT_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace ft
