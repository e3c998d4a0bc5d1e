// Routing of a mixture of experts whose scores are sigmoids, and the gated activation of the chosen experts.
//
// Router: s_e = sigmoid(z_e) from 32-bit logits.  The experts form `n_groups` equal groups of neighbours; a
// group's score is the sum of its two largest s (of its only one, in groups of one); only experts of the
// `keep` best groups can be chosen; the `top` largest s among those are chosen; their weights are s divided
// by the sum of the chosen s (+ 1e-20).  Ties go to the lower index.  A shared expert's gate, sigmoid of one
// more logit, is written as one more column.  All of it is 32-bit.
//
// Output: a dense row of weights per token, [experts (+ 1)], zero for the experts that were not chosen, and
// the chosen experts with their weights as lists [top].
#include "common.cuh"

#define RE_MAX_EXPERTS 1024

__device__ __forceinline__ void re_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// one warp a token
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ z, int ld, float* __restrict__ dense, int* __restrict__ pick,
             float* __restrict__ pick_w, int N, int E, int n_groups, int keep, int top, int shared_gate) {
    mv_pdl_begin();
    extern __shared__ float re_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    float* s = re_smem + (size_t)warp * (E + n_groups);       // scores; -1 once taken or not allowed
    float* gs = s + E;                                        // group scores
    const float* zr = z + (size_t)n * ld;
    const int cols = E + (shared_gate ? 1 : 0);
    float* dr = dense + (size_t)n * cols;
    for (int e = lane; e < E; e += 32) {
        s[e] = 1.0f / (1.0f + expf(-zr[e]));
        dr[e] = 0.f;
    }
    if (shared_gate && lane == 0) dr[E] = 1.0f / (1.0f + expf(-zr[E]));
    __syncwarp();
    const int per = E / n_groups;
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -1.f, b = -1.f;                          // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = s[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = a + (per > 1 ? b : 0.f);
        }
        __syncwarp();
        // the best `keep` groups keep a score >= 0 in gs; then the others' experts are struck out
        for (int r = 0; r < keep; ++r) {
            float v = -1.f; int i = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32)
                if (gs[g] > v) { v = gs[g]; i = g; }
            re_argmax(v, i);
            if (lane == 0) gs[i] = -2.f;                       // chosen
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != -2.f) s[e] = -1.f;
        __syncwarp();
    }
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
        float v = -1.f; int i = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (s[e] > v) { v = s[e]; i = e; }
        re_argmax(v, i);
        sum += v;
        if (lane == 0) {
            pick[(size_t)n * top + r] = i;
            pick_w[(size_t)n * top + r] = v;
            s[i] = -1.f;
        }
        __syncwarp();
    }
    const float inv = 1.0f / (sum + 1e-20f);
    if (lane < top) {
        // (top <= 32 is checked by the host)
        const float w = pick_w[(size_t)n * top + lane] * inv;
        pick_w[(size_t)n * top + lane] = w;
        dr[pick[(size_t)n * top + lane]] = w;
    }
}

// z [N, >= E (+ 1)] with row stride ld; dense [N, E (+ 1)]; pick, pick_w [N, top].
MV_API int mv_route(const float* z, int ld, float* dense, int* pick, float* pick_w, int N, int E, int n_groups,
                    int keep, int top, int shared_gate, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E < 1 || E > RE_MAX_EXPERTS || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups || top < 1 ||
        top > 32 || top > keep * (E / n_groups))
        return (int)cudaErrorInvalidValue;
    const int warps = 4;
    const size_t smem = sizeof(float) * warps * (size_t)(E + n_groups);
    mv_launch(route_kernel, (N + warps - 1) / warps, warps * 32, smem, stream, z, ld, dense, pick, pick_w, N, E,
              n_groups, keep, top, shared_gate);
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// hid[n, c] = w[n, expert(c)] * silu(gate[n, c]) * up[n, c] over the columns of all experts laid end to end
// (expert e owns [e * ff, (e + 1) * ff), a shared expert the `shared_ff` columns after them, with the weight of
// column E).  gu [N, 2 * F]: all gates, then all ups.  Where the weight is zero nothing is computed.
template <typename TO>
__global__ void __launch_bounds__(256)
routed_glu_kernel(const float* __restrict__ gu, const float* __restrict__ dense, TO* __restrict__ hid, long long total,
                  int F, int E, int ff, int cols) {
    mv_pdl_begin();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long n = idx / F;
    const int c = (int)(idx - n * F);
    const int e = c < E * ff ? c / ff : E;
    const float w = dense[n * cols + e];
    float out = 0.f;
    if (w != 0.f) {
        const float g = gu[n * 2 * F + c], u = gu[n * 2 * F + F + c];
        out = w * (g / (1.0f + expf(-g))) * u;
    }
    hid[idx] = mv_from_f32<TO>(out);
}

MV_API int mv_routed_glu(const float* gu, const float* dense, void* hid, int hid_dtype, int N, int E, int ff,
                         int shared_ff, cudaStream_t stream) {
    if (N <= 0) return 0;
    const int F = E * ff + shared_ff, cols = E + (shared_ff ? 1 : 0);
    const long long total = (long long)N * F;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (hid_dtype == MV_DT_BF16)
        mv_launch(routed_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, gu, dense, (__nv_bfloat16*)hid, total, F, E,
                  ff, cols);
    else
        mv_launch(routed_glu_kernel<float>, blocks, 256, 0, stream, gu, dense, (float*)hid, total, F, E, ff, cols);
    return mv_launch_status();
}
