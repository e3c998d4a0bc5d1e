// Linear attention with a decaying matrix state, one head at a time:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: dk x dv, a_t: a factor per key channel)
//     o_t = S_t^T q_t
//
// The state lives in 32-bit floats per sequence slot and is carried from step to step; a step
// brings any number of next tokens for each of its sequences.  Everything here is 32-bit: the
// decay, the state, the sums.  Two ways to say the decay cover the designs in use:
//   * per token and key channel from logits z: a = sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau)
//     (gated linear attention), or
//   * one constant per head (lightning attention).
// q, k and v come as 32-bit rows of a projection (any row stride, any column offset); an
// activation (none or silu) and a factor on q are applied as they are read.
//
// Work: a block is (16 value columns, head, sequence) and walks the sequence's tokens in order.
// A value column is owned by 8 lanes, lane p holding the state's rows p, p+8, p+16, ... of that
// column in registers; the state is stored [slot][head][dv][dk], so these 8 lanes read 32
// contiguous bytes.  Tokens come through shared memory eight at a time.  The order of every sum
// depends on nothing but dk, so a prompt gives the same numbers however it is cut into steps.
#include "common.cuh"

#define DS_COLS 16
#define DS_PART 8
#define DS_CHUNK 8

__device__ __forceinline__ float ds_silu(float x) { return x / (1.0f + expf(-x)); }
// log(sigmoid(z)) without overflow: min(z, 0) - log1p(exp(-|z|))
__device__ __forceinline__ float ds_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <int R>
__global__ void __launch_bounds__(DS_COLS * DS_PART)
decay_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                  const float* __restrict__ v, int ldv, const float* __restrict__ z, int ldz,
                  const float* __restrict__ head_decay, float inv_tau, float q_scale, int act,
                  float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                  float* __restrict__ o, int n_heads, int dk, int dv) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    float* qs = smem;                           // [DS_CHUNK][dk]
    float* ks = qs + DS_CHUNK * dk;
    float* as = ks + DS_CHUNK * dk;
    float* vs = as + DS_CHUNK * dk;             // [DS_CHUNK][DS_COLS]
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, p = tid & (DS_PART - 1), jl = tid >> 3;
    const int j = tile * DS_COLS + jl;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const int slot = mv_read_slot(slots[b]);
    float* srow = state + (((size_t)slot * n_heads + h) * dv + (j < dv ? j : 0)) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = p + DS_PART * r;
        S[r] = (j < dv && i < dk) ? srow[i] : 0.f;
    }
    const float hd = head_decay ? head_decay[h] : 1.f;
    for (int c0 = 0; c0 < len; c0 += DS_CHUNK) {
        const int nt = min(DS_CHUNK, len - c0);
        __syncthreads();
        for (int idx = tid; idx < nt * dk; idx += DS_COLS * DS_PART) {
            const int t = idx / dk, i = idx - t * dk;
            const size_t row = (size_t)(row0 + c0 + t);
            float qv = q[row * ldq + (size_t)h * dk + i], kv = k[row * ldk + (size_t)h * dk + i];
            if (act) { qv = ds_silu(qv); kv = ds_silu(kv); }
            qs[t * dk + i] = qv * q_scale;
            ks[t * dk + i] = kv;
            as[t * dk + i] = z ? expf(ds_log_sigmoid(z[row * ldz + (size_t)h * dk + i]) * inv_tau) : hd;
        }
        for (int idx = tid; idx < nt * DS_COLS; idx += DS_COLS * DS_PART) {
            const int t = idx / DS_COLS, c = idx - t * DS_COLS, col = tile * DS_COLS + c;
            float vv = col < dv ? v[(size_t)(row0 + c0 + t) * ldv + (size_t)h * dv + col] : 0.f;
            vs[idx] = act ? ds_silu(vv) : vv;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = vs[t * DS_COLS + jl];
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            const float* at = as + t * dk;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + DS_PART * r;
                if (i < dk) {
                    S[r] = fmaf(at[i], S[r], kt[i] * vj);
                    acc = fmaf(S[r], qt[i], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (p == 0 && j < dv) o[(size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv + j] = acc;
        }
    }
    if (j < dv && mv_slot_ok(slots[b])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = p + DS_PART * r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

MV_GUARD_SETTER(decay_scan)

// q, k [N, >= n_heads * dk], v [N, >= n_heads * dv] with row strides ldq, ldk, ldv (elements);
// z: decay logits [N, >= n_heads * dk] with stride ldz, or null, then head_decay [n_heads];
// state [slots][n_heads][dv][dk]; slots [n_seqs]; cu [n_seqs + 1]; o [N, n_heads * dv] dense.
MV_API int mv_decay_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                         const float* z, int ldz, const float* head_decay, float inv_tau, float q_scale, int act,
                         float* state, const int* slots, const int* cu, float* o, int n_seqs, int n_heads, int dk,
                         int dv, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || (!z && !head_decay)) return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + DS_COLS - 1) / DS_COLS, n_heads, n_seqs);
    const size_t smem = (size_t)DS_CHUNK * (3 * dk + DS_COLS) * sizeof(float);
    if (dk <= 64)
        mv_launch(decay_scan_kernel<8>, grid, DS_COLS * DS_PART, smem, stream, q, ldq, k, ldk, v, ldv, z, ldz,
                  head_decay, inv_tau, q_scale, act, state, slots, cu, o, n_heads, dk, dv);
    else if (dk <= 128)
        mv_launch(decay_scan_kernel<16>, grid, DS_COLS * DS_PART, smem, stream, q, ldq, k, ldk, v, ldv, z, ldz,
                  head_decay, inv_tau, q_scale, act, state, slots, cu, o, n_heads, dk, dv);
    else
        mv_launch(decay_scan_kernel<32>, grid, DS_COLS * DS_PART, smem, stream, q, ldq, k, ldk, v, ldv, z, ldz,
                  head_decay, inv_tau, q_scale, act, state, slots, cu, o, n_heads, dk, dv);
    return mv_launch_status();
}
