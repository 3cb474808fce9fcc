// Linear attention with a fixed decay per head (a recurrence over a state of fixed size instead of a softmax over
// cached keys), and the gated norm that follows it.
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S: [dim, vdim] per (request, head), fp32, zero at admission
//   o_t = S_t^T q_t                            no other scale
//
// The columns of S do not depend on one another, so a warp owns eight of them for one (request, head) and walks
// the request's tokens of the step in order: a lane holds rows lane, lane + 32, ... of its eight columns in
// registers, updates them with fp32 FMAs, and the eight dot products with q are summed over the warp.  No barrier,
// no shared memory; a step of single tokens and a long portion of a prompt are the same loop.  The state lies
// transposed in memory, [slot, head, vdim, dim], so that a warp reads and writes whole rows of it.
// q, k, v may be passed through SiLU on the way in (`silu`), in fp32 whatever the storage type.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LA_COLS = 8;
constexpr int LA_WARPS = 4;

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int RPL>  // RPL rows of the state per lane: dim <= 32 * RPL
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_scan_kernel(
    const T* qkv, int ld, int q_off, int k_off, int v_off, float* __restrict__ out, int ldo, float* state,
    const float* __restrict__ decay, const int* __restrict__ seq_q_start, const int* __restrict__ seq_state_slot,
    int heads, int dim, int vdim, int silu, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int col0 = (blockIdx.x * LA_WARPS + warp) * LA_COLS;
    if (col0 >= vdim) return;
    const int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    if (row1 <= row0) return;
    const float lam = decay[h];
    float* st = state + (((size_t)seq_state_slot[seq] * heads + h) * vdim + col0) * dim;
    float S[LA_COLS][RPL];
#pragma unroll
    for (int c = 0; c < LA_COLS; ++c)
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            S[c][r] = (col0 + c < vdim && i < dim) ? st[(size_t)c * dim + i] : 0.0f;
        }
    for (int t = row0; t < row1; ++t) {
        const T* row = qkv + (size_t)t * ld;
        float kk[RPL], qq[RPL], vv[LA_COLS];
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            float a = i < dim ? to_float(row[k_off + h * dim + i]) : 0.0f;
            float b = i < dim ? to_float(row[q_off + h * dim + i]) : 0.0f;
            kk[r] = silu ? silu_f(a) : a;
            qq[r] = silu ? silu_f(b) : b;
        }
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c) {
            const float a = col0 + c < vdim ? to_float(row[v_off + h * vdim + col0 + c]) : 0.0f;
            vv[c] = silu ? silu_f(a) : a;
        }
        float o[LA_COLS];
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c) {
            float acc = 0.0f;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                S[c][r] = fmaf(kk[r], vv[c], lam * S[c][r]);
                acc = fmaf(S[c][r], qq[r], acc);
            }
            o[c] = warp_sum(acc);
        }
        float mine = 0.0f;
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c)
            if (lane == c) mine = o[c];
        if (lane < LA_COLS && col0 + lane < vdim) out[(size_t)t * ldo + h * vdim + col0 + lane] = mine;
    }
    if (write_state) {
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c)
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int i = lane + 32 * r;
                if (col0 + c < vdim && i < dim) st[(size_t)c * dim + i] = S[c][r];
            }
    }
}

// out[t, i] = (o[t, i] / sqrt(mean_i(o[t, :]^2) + eps)) * w[i] * sigmoid(g[t, i]); o fp32, g and out in the
// activations' type.  A block per row.
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const float* o, int ldi, const T* g, int ldg,
                                                            const float* __restrict__ w, T* __restrict__ out, int ldo,
                                                            int n, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float* orow = o + (size_t)t * ldi;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = orow[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    const T* grow = g + (size_t)t * ldg;
    T* dst = out + (size_t)t * ldo;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-to_float(grow[i])));
        dst[i] = from_float<T>(((orow[i] * inv) * w[i]) * gate);
    }
}

template <typename T>
int launch_scan(const void* qkv, int ld, int q_off, int k_off, int v_off, float* out, int ldo, float* state,
                const float* decay, const int* seq_q_start, const int* seq_state_slot, int seqs, int heads, int dim,
                int vdim, int silu, int write_state, cudaStream_t s) {
    const dim3 grid((vdim + LA_COLS * LA_WARPS - 1) / (LA_COLS * LA_WARPS), heads, seqs), block(LA_WARPS * 32);
#define FERRIS_LA_LAUNCH(RPL)                                                                                          \
    ferris_launch(linear_attention_scan_kernel<T, RPL>, grid, block, 0, s, (const T*)qkv, ld, q_off, k_off, v_off, out, \
                  ldo, state, decay, seq_q_start, seq_state_slot, heads, dim, vdim, silu, write_state)
    if (dim <= 32)
        FERRIS_LA_LAUNCH(1);
    else if (dim <= 64)
        FERRIS_LA_LAUNCH(2);
    else if (dim <= 128)
        FERRIS_LA_LAUNCH(4);
    else
        FERRIS_LA_LAUNCH(8);
#undef FERRIS_LA_LAUNCH
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// qkv: rows of ld elements holding q heads at q_off, k heads at k_off (heads x dim each) and v heads at v_off
// (heads x vdim), head by head; out: fp32 [tokens, heads x vdim] rows ldo apart; state: fp32 [slots, heads, vdim, dim];
// decay: fp32 [heads].  The rows of request s are seq_q_start[s] .. seq_q_start[s + 1] - 1, in order.
FERRIS_API int ferris_linear_attention(const void* qkv, int ld, int q_off, int k_off, int v_off, int dtype, float* out,
                                       int ldo, float* state, const float* decay, const int* seq_q_start,
                                       const int* seq_state_slot, int seqs, int heads, int dim, int vdim, int silu,
                                       int write_state, void* stream) {
    if (seqs <= 0) return FERRIS_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 256) FERRIS_REFUSE("linear attention: heads=%d dim=%d vdim=%d (dim at most 256)", heads, dim, vdim);
    if (heads > 65535 || seqs > 65535) FERRIS_REFUSE("linear attention: %d heads of %d requests are more than one launch takes", heads, seqs);
    if (!state || !decay) FERRIS_REFUSE("linear attention: no state or no decay");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        return launch_scan<float>(qkv, ld, q_off, k_off, v_off, out, ldo, state, decay, seq_q_start, seq_state_slot, seqs, heads, dim, vdim, silu, write_state, s);
    if (dtype == FERRIS_BF16)
        return launch_scan<bf16>(qkv, ld, q_off, k_off, v_off, out, ldo, state, decay, seq_q_start, seq_state_slot, seqs, heads, dim, vdim, silu, write_state, s);
    FERRIS_REFUSE("linear attention: unknown dtype %d", dtype);
}

FERRIS_API int ferris_gated_rmsnorm(const float* o, int ldi, const void* g, int ldg, const float* w, void* out, int ldo,
                                    int dtype, int rows, int n, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (n <= 0) FERRIS_REFUSE("gated rmsnorm: %d columns", n);
    const int threads = n >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(gated_rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, s, o, ldi, (const float*)g, ldg, w, (float*)out, ldo, n, eps);
    else if (dtype == FERRIS_BF16)
        ferris_launch(gated_rmsnorm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, o, ldi, (const bf16*)g, ldg, w, (bf16*)out, ldo, n, eps);
    else
        FERRIS_REFUSE("gated rmsnorm: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
