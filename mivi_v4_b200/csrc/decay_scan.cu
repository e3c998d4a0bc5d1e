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

// ---------------------------------------------------------------------------------------------
// The same recurrence for steps that bring many tokens a sequence, in chunks of DC_CHUNK tokens:
// what a token reads from the tokens of its own chunk and what it reads from the state before the
// chunk are separated, so that only the state's hand-over from chunk to chunk is sequential.  With
// c_t the sum of log a over the chunk's tokens up to t (per key channel; all of it <= 0),
//
//     o_t  = sum_i q_t,i e^(c_t,i) S0[i, :]  +  sum_{s <= t} P[t, s] v_s ,
//     P[t, s] = sum_i q_t,i k_s,i e^(c_t,i - c_s,i) ,
//     S_end[i, :] = e^(c_last,i) S0[i, :] + sum_s k_s,i e^(c_last,i - c_s,i) v_s .
//
// Every exponent is a difference of cumulative logarithms taken the right way round, so every factor
// lies in (0, 1]: nothing overflows however small a decay is.  All of it is float32 on the CUDA cores.
// The first kernel prepares, per (sequence, head, chunk), the decayed q and k, the chunk's total decay
// and P; the second walks a sequence's chunks with the state in registers.
//
// Chunks are numbered floor(cu[b] / DC_CHUNK) + b + c for chunk c of the step's sequence b: distinct
// numbers below N / DC_CHUNK + n_seqs + 1 that need nothing from the host.
#define DC_CHUNK 32
#define DC_COLS 16
#define DC_THREADS 256            // the preparing kernel
#define DC_SCAN_THREADS 512       // the scanning kernel: 32 half-warps
#define DC_GROUPS (DC_SCAN_THREADS / 16)
// a group's shares of a chunk's outputs, padded by half a row of banks: the two groups of a warp then store into
// different banks
#define DC_RED_STRIDE (DC_CHUNK * DC_COLS + 16)

__global__ void __launch_bounds__(DC_THREADS)
decay_chunk_prepare_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                           const float* __restrict__ z, int ldz, const float* __restrict__ head_decay, float inv_tau,
                           float q_scale, int act, const int* __restrict__ cu, float* __restrict__ qd,
                           float* __restrict__ kd, float* __restrict__ ed, float* __restrict__ P, int n_heads, int dk) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    const int lds = dk + 1;                         // odd row stride: rows of different tokens fall into different banks
    float* cs = smem;                               // [DC_CHUNK][lds] cumulative log decay
    float* qa = cs + DC_CHUNK * lds;                // activated, scaled q
    float* ka = qa + DC_CHUNK * lds;                // activated k
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (c * DC_CHUNK >= len) return;
    const int nt = min(DC_CHUNK, len - c * DC_CHUNK);
    const int first = row0 + c * DC_CHUNK;
    const int chunk = row0 / DC_CHUNK + b + c;
    const int tid = threadIdx.x;
    // a decay of exactly 0 has no logarithm; e^-80 stands in for it (what is left of the state then lies 35
    // decimal places down)
    const float log_hd = head_decay ? fmaxf(logf(head_decay[h]), -80.f) : 0.f;
    for (int idx = tid; idx < nt * dk; idx += DC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        const size_t row = (size_t)(first + t);
        float qv = q[row * ldq + (size_t)h * dk + i], kv = k[row * ldk + (size_t)h * dk + i];
        if (act) { qv = ds_silu(qv); kv = ds_silu(kv); }
        qa[t * lds + i] = qv * q_scale;
        ka[t * lds + i] = kv;
        cs[t * lds + i] = z ? ds_log_sigmoid(z[row * ldz + (size_t)h * dk + i]) * inv_tau : log_hd;
    }
    __syncthreads();
    for (int i = tid; i < dk; i += DC_THREADS) {
        float run = 0.f;
        for (int t = 0; t < nt; ++t) {
            run += cs[t * lds + i];
            cs[t * lds + i] = run;
        }
    }
    __syncthreads();
    const int width = n_heads * dk;
    for (int idx = tid; idx < nt * dk; idx += DC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        const size_t at = (size_t)(first + t) * width + (size_t)h * dk + i;
        qd[at] = qa[t * lds + i] * expf(cs[t * lds + i]);
        kd[at] = ka[t * lds + i] * expf(cs[(nt - 1) * lds + i] - cs[t * lds + i]);
    }
    for (int i = tid; i < dk; i += DC_THREADS) ed[(size_t)chunk * width + (size_t)h * dk + i] = expf(cs[(nt - 1) * lds + i]);
    float* Pc = P + ((size_t)chunk * n_heads + h) * DC_CHUNK * DC_CHUNK;
    for (int p = tid; p < DC_CHUNK * DC_CHUNK; p += DC_THREADS) {
        const int t = p / DC_CHUNK, s = p - t * DC_CHUNK;
        float sum = 0.f;
        if (s <= t && t < nt) {
            const float* ct = cs + t * lds;
            const float* cq = cs + s * lds;
            const float* qt = qa + t * lds;
            const float* kt = ka + s * lds;
            if (z) {
                for (int i = 0; i < dk; ++i) sum = fmaf(qt[i] * kt[i], expf(ct[i] - cq[i]), sum);
            } else {
                // one decay for all of the head's channels: its power is a factor of the whole sum
                for (int i = 0; i < dk; ++i) sum = fmaf(qt[i], kt[i], sum);
                sum *= expf(ct[0] - cq[0]);
            }
        }
        Pc[p] = sum;
    }
}

// A block is 16 value columns of one head of one sequence; its 16 warps are 32 half-warps, each holding RH key
// channels of every column in registers (dk <= 32 * RH): lane & 15 is the column, the half-warp the channel group.
template <int RH>
__global__ void __launch_bounds__(DC_SCAN_THREADS)
decay_chunk_scan_kernel(const float* __restrict__ qd, const float* __restrict__ kd, const float* __restrict__ ed,
                        const float* __restrict__ P, const float* __restrict__ v, int ldv, int act,
                        float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                        float* __restrict__ o, int n_heads, int dk, int dv) {
    mv_pdl_begin();
    constexpr int DKP = DC_GROUPS * RH;
    extern __shared__ __align__(16) float smem[];
    float* qt = smem;                               // [DC_CHUNK][DKP], zero beyond dk
    float* kt = qt + DC_CHUNK * DKP;
    float* vt = kt + DC_CHUNK * DKP;                // [DC_CHUNK][DC_COLS]
    float* pt = vt + DC_CHUNK * DC_COLS;            // [DC_CHUNK][DC_CHUNK]
    float* et = pt + DC_CHUNK * DC_CHUNK;           // [DKP]
    float* red = et + DKP;                          // [DC_GROUPS][DC_RED_STRIDE]: [DC_CHUNK][DC_COLS] a group
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, col = tid & 15, grp = tid >> 4;
    const int j = tile * DC_COLS + col;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const int slot = mv_read_slot(slots[b]);
    const int width = n_heads * dk;
    float* srow = state + (((size_t)slot * n_heads + h) * dv + (j < dv ? j : 0)) * dk;
    float S[RH];
#pragma unroll
    for (int r = 0; r < RH; ++r) {
        const int i = grp * RH + r;
        S[r] = (j < dv && i < dk) ? srow[i] : 0.f;
    }
    const int n_chunks = (len + DC_CHUNK - 1) / DC_CHUNK;
    // A chunk's rows are requested into registers while the chunk before is worked on, and go to shared
    // memory when that one is done: per thread IT values of the decayed q and of the decayed k, 2 of v, 4 of P
    // and at most one of the chunk's total decay.
    constexpr int IT = DC_CHUNK * DKP / DC_SCAN_THREADS;
    static_assert(DC_CHUNK * DC_COLS == DC_SCAN_THREADS && DC_CHUNK * DC_CHUNK % DC_SCAN_THREADS == 0 && DKP <= DC_SCAN_THREADS,
                  "a thread requests one value of v, whole rounds of P and at most one of the total decay");
    float rq[IT], rk[IT], rv[DC_CHUNK * DC_COLS / DC_SCAN_THREADS], rp[DC_CHUNK * DC_CHUNK / DC_SCAN_THREADS], re = 0.f;
    auto request = [&](int c) {
        const int nt = min(DC_CHUNK, len - c * DC_CHUNK);
        const int first = row0 + c * DC_CHUNK;
        const int chunk = row0 / DC_CHUNK + b + c;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int idx = tid + it * DC_SCAN_THREADS, t = idx / DKP, i = idx - t * DKP;
            const bool in = t < nt && i < dk;
            const size_t at = in ? (size_t)(first + t) * width + (size_t)h * dk + i : 0;
            rq[it] = in ? qd[at] : 0.f;
            rk[it] = in ? kd[at] : 0.f;
        }
#pragma unroll
        for (int it = 0; it < DC_CHUNK * DC_COLS / DC_SCAN_THREADS; ++it) {
            const int idx = tid + it * DC_SCAN_THREADS, t = idx / DC_COLS, cc = tile * DC_COLS + (idx - t * DC_COLS);
            const float vv = (t < nt && cc < dv) ? v[(size_t)(first + t) * ldv + (size_t)h * dv + cc] : 0.f;
            rv[it] = act ? ds_silu(vv) : vv;
        }
        const float* Pc = P + ((size_t)chunk * n_heads + h) * DC_CHUNK * DC_CHUNK;
#pragma unroll
        for (int it = 0; it < DC_CHUNK * DC_CHUNK / DC_SCAN_THREADS; ++it) rp[it] = Pc[tid + it * DC_SCAN_THREADS];
        if (tid < DKP) re = tid < dk ? ed[(size_t)chunk * width + (size_t)h * dk + tid] : 0.f;
    };
    request(0);
    for (int c = 0; c < n_chunks; ++c) {
        const int nt = min(DC_CHUNK, len - c * DC_CHUNK);
        const int first = row0 + c * DC_CHUNK;
        __syncthreads();                            // the chunk before is done with shared memory
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            qt[tid + it * DC_SCAN_THREADS] = rq[it];
            kt[tid + it * DC_SCAN_THREADS] = rk[it];
        }
#pragma unroll
        for (int it = 0; it < DC_CHUNK * DC_COLS / DC_SCAN_THREADS; ++it) vt[tid + it * DC_SCAN_THREADS] = rv[it];
#pragma unroll
        for (int it = 0; it < DC_CHUNK * DC_CHUNK / DC_SCAN_THREADS; ++it) pt[tid + it * DC_SCAN_THREADS] = rp[it];
        if (tid < DKP) et[tid] = re;
        __syncthreads();
        if (c + 1 < n_chunks) request(c + 1);
        // what the chunk's tokens read from the state before the chunk: this half-warp's key channels
#pragma unroll 4
        for (int t = 0; t < DC_CHUNK; ++t) {
            const float4* q4 = reinterpret_cast<const float4*>(qt + t * DKP + grp * RH);
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RH; r += 4) {
                const float4 x = q4[r >> 2];
                acc = fmaf(x.x, S[r], acc); acc = fmaf(x.y, S[r + 1], acc);
                acc = fmaf(x.z, S[r + 2], acc); acc = fmaf(x.w, S[r + 3], acc);
            }
            red[grp * DC_RED_STRIDE + t * DC_COLS + col] = acc;
        }
        // the state after the chunk
#pragma unroll
        for (int r = 0; r < RH; ++r) S[r] *= et[grp * RH + r];
#pragma unroll 4
        for (int s = 0; s < DC_CHUNK; ++s) {
            const float vj = vt[s * DC_COLS + col];
            const float4* k4 = reinterpret_cast<const float4*>(kt + s * DKP + grp * RH);
#pragma unroll
            for (int r = 0; r < RH; r += 4) {
                const float4 x = k4[r >> 2];
                S[r] = fmaf(x.x, vj, S[r]); S[r + 1] = fmaf(x.y, vj, S[r + 1]);
                S[r + 2] = fmaf(x.z, vj, S[r + 2]); S[r + 3] = fmaf(x.w, vj, S[r + 3]);
            }
        }
        __syncthreads();
        // outputs: the groups' shares in a fixed order, then the chunk's own tokens
        for (int idx = tid; idx < nt * DC_COLS; idx += DC_SCAN_THREADS) {
            const int t = idx / DC_COLS, cc = idx - t * DC_COLS;
            float sum = 0.f;
#pragma unroll
            for (int g = 0; g < DC_GROUPS; ++g) sum += red[g * DC_RED_STRIDE + t * DC_COLS + cc];
            for (int s = 0; s <= t; ++s) sum = fmaf(pt[t * DC_CHUNK + s], vt[s * DC_COLS + cc], sum);
            if (tile * DC_COLS + cc < dv) o[(size_t)(first + t) * n_heads * dv + (size_t)h * dv + tile * DC_COLS + cc] = sum;
        }
    }
    if (j < dv && mv_slot_ok(slots[b])) {
#pragma unroll
        for (int r = 0; r < RH; ++r) {
            const int i = grp * RH + r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

template <int RH>
static int decay_chunk_scan_launch(dim3 grid, cudaStream_t stream, const float* qd, const float* kd, const float* ed,
                                   const float* P, const float* v, int ldv, int act, float* state, const int* slots,
                                   const int* cu, float* o, int n_heads, int dk, int dv) {
    const size_t smem = sizeof(float) * ((size_t)2 * DC_CHUNK * DC_GROUPS * RH + DC_CHUNK * DC_COLS + DC_CHUNK * DC_CHUNK +
                                         DC_GROUPS * RH + DC_GROUPS * DC_RED_STRIDE);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(decay_chunk_scan_kernel<RH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    mv_launch(decay_chunk_scan_kernel<RH>, grid, DC_SCAN_THREADS, smem, stream, qd, kd, ed, P, v, ldv, act, state, slots, cu, o,
              n_heads, dk, dv);
    return mv_launch_status();
}

// How many chunks the scratch of a step of N tokens in n_seqs sequences must hold.
MV_API int mv_decay_chunks(int N, int n_seqs) { return N / DC_CHUNK + n_seqs + 1; }

// Arguments as mv_decay_scan, plus the longest sequence's tokens (max_len) and scratch: qd, kd [N, n_heads * dk],
// ed [chunks, n_heads * dk], P [chunks, n_heads, DC_CHUNK, DC_CHUNK] with chunks = mv_decay_chunks(N, n_seqs).
MV_API int mv_decay_scan_chunked(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                 const float* z, int ldz, const float* head_decay, float inv_tau, float q_scale, int act,
                                 float* state, const int* slots, const int* cu, float* o, float* qd, float* kd, float* ed,
                                 float* P, int n_seqs, int max_len, int n_heads, int dk, int dv, cudaStream_t stream) {
    if (n_seqs <= 0 || max_len <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || (!z && !head_decay)) return (int)cudaErrorInvalidValue;
    const size_t smem_a = sizeof(float) * (size_t)3 * DC_CHUNK * (dk + 1);
    static size_t attr_a = 0;
    if (smem_a > attr_a) {
        cudaFuncSetAttribute(decay_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        attr_a = smem_a;
    }
    mv_launch(decay_chunk_prepare_kernel, dim3((max_len + DC_CHUNK - 1) / DC_CHUNK, n_heads, n_seqs), DC_THREADS, smem_a,
              stream, q, ldq, k, ldk, z, ldz, head_decay, inv_tau, q_scale, act, cu, qd, kd, ed, P, n_heads, dk);
    int code = mv_launch_status();
    if (code) return code;
    const dim3 grid((dv + DC_COLS - 1) / DC_COLS, n_heads, n_seqs);
    if (dk <= 128) return decay_chunk_scan_launch<4>(grid, stream, qd, kd, ed, P, v, ldv, act, state, slots, cu, o, n_heads, dk, dv);
    return decay_chunk_scan_launch<8>(grid, stream, qd, kd, ed, P, v, ldv, act, state, slots, cu, o, n_heads, dk, dv);
}
