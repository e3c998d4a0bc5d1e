// A matrix state per head that decays by ONE factor per token and head:
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T          (S: dk x dv; a_t, b_t scalars of the token and head)
//     o_t = S_t^T q_t  (+ skip_h v_t)
//
// which is the recurrence of a selective state space layer (a_t = e^(A dt_t), b_t = dt_t, k = B, q = C,
// v = x, skip = D) and of a matrix memory with exponential gates (a_t = e^(f_t + m_(t-1) - m_t),
// b_t = e^(i_t - m_t), m the running maximum of the log gates).  The matrix memory also keeps a
// normalizer n_t = a_t n_(t-1) + b_t k_t, stored as one more value column of the state, and divides:
// o_t <- o_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).
//
// The state lives in 32-bit floats per sequence slot, [slot][head][dv (+1)][dk]; log a_t and b_t come as
// 32-bit numbers per token and head; q, k, v are 32-bit rows (any row stride, any column offset); several
// heads may share one q and k (a group).  Everything is computed in 32-bit.
//
// Work of the token-by-token kernel: a block is (16 value columns, head, sequence) and walks the
// sequence's tokens in order; a value column is owned by 8 lanes, lane p holding rows p, p+8, ... of that
// column in registers.  With a normalizer every block carries that column too (as a 17th group of lanes),
// so that it can divide without waiting for another block; the block of the first tile stores it.  The
// order of every sum depends on nothing but dk, so a prompt gives the same numbers however it is cut.
#include "common.cuh"

#define SS_COLS 16
#define SS_PART 8
#define SS_CHUNK 8

template <int R>
__global__ void __launch_bounds__(SS_COLS * SS_PART + 32)
scalar_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                   const float* __restrict__ v, int ldv, const float* __restrict__ log_a, int ld_a,
                   const float* __restrict__ b_in, int ld_b, const float* __restrict__ skip,
                   const float* __restrict__ m_tok, float q_scale, float* __restrict__ state,
                   const int* __restrict__ slots, const int* __restrict__ cu, float* __restrict__ o, int n_heads,
                   int heads_per_group, int dk, int dv, int normalizer) {
    mv_pdl_begin();
    extern __shared__ float smem[];
    float* qs = smem;                           // [SS_CHUNK][dk]
    float* ks = qs + SS_CHUNK * dk;             // [SS_CHUNK][dk], already times b_t
    float* vs = ks + SS_CHUNK * dk;             // [SS_CHUNK][SS_COLS]
    float* as = vs + SS_CHUNK * SS_COLS;        // [SS_CHUNK] decay factors
    float* ms = as + SS_CHUNK;                  // [SS_CHUNK] e^(-m_t)
    float* acc_s = ms + SS_CHUNK;               // [SS_CHUNK][SS_COLS + 1]
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, p = tid & (SS_PART - 1), jl = tid >> 3;
    const int n_threads = blockDim.x;
    const bool is_n = jl == SS_COLS;                          // the normalizer's lanes
    const int cols = dv + (normalizer ? 1 : 0);
    const int j = jl >= SS_COLS ? dv : tile * SS_COLS + jl;
    const bool live = is_n ? normalizer != 0 : (jl < SS_COLS && j < dv);    // a whole last warp: its other lanes idle
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const int slot = mv_read_slot(slots[b]);
    const size_t qk_off = (size_t)(h / heads_per_group) * dk;
    float* srow = state + (((size_t)slot * n_heads + h) * cols + (live ? j : 0)) * dk;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = p + SS_PART * r;
        S[r] = (live && i < dk) ? srow[i] : 0.f;
    }
    const float sk = skip ? skip[h] : 0.f;
    for (int c0 = 0; c0 < len; c0 += SS_CHUNK) {
        const int nt = min(SS_CHUNK, len - c0);
        __syncthreads();
        if (tid < nt) {
            const size_t row = (size_t)(row0 + c0 + tid);
            as[tid] = expf(log_a[row * ld_a + h]);
            ms[tid] = m_tok ? expf(-m_tok[row * n_heads + h]) : 0.f;
        }
        for (int idx = tid; idx < nt * dk; idx += n_threads) {
            const int t = idx / dk, i = idx - t * dk;
            const size_t row = (size_t)(row0 + c0 + t);
            qs[idx] = q[row * ldq + qk_off + i] * q_scale;
            ks[idx] = k[row * ldk + qk_off + i] * b_in[row * ld_b + h];
        }
        for (int idx = tid; idx < nt * SS_COLS; idx += n_threads) {
            const int t = idx / SS_COLS, c = idx - t * SS_COLS, col = tile * SS_COLS + c;
            vs[idx] = col < dv ? v[(size_t)(row0 + c0 + t) * ldv + (size_t)h * dv + col] : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = is_n ? 1.f : vs[t * SS_COLS + (jl < SS_COLS ? jl : 0)];
            const float a = as[t];
            const float* qt = qs + t * dk;
            const float* kt = ks + t * dk;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = p + SS_PART * r;
                if (i < dk) {
                    S[r] = fmaf(a, S[r], kt[i] * vj);
                    acc = fmaf(S[r], qt[i], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (p == 0 && jl <= SS_COLS) acc_s[t * (SS_COLS + 1) + jl] = acc + (is_n ? 0.f : sk * vj);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * SS_COLS; idx += n_threads) {
            const int t = idx / SS_COLS, c = idx - t * SS_COLS, col = tile * SS_COLS + c;
            if (col >= dv) continue;
            float val = acc_s[t * (SS_COLS + 1) + c];
            if (normalizer) val = val / (fmaxf(fabsf(acc_s[t * (SS_COLS + 1) + SS_COLS]), ms[t]) + 1e-6f);
            o[(size_t)(row0 + c0 + t) * n_heads * dv + (size_t)h * dv + col] = val;
        }
    }
    if (live && (!is_n || tile == 0) && mv_slot_ok(slots[b])) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = p + SS_PART * r;
            if (i < dk) srow[i] = S[r];
        }
    }
}

MV_GUARD_SETTER(scalar_scan)

// q, k [N, >= (n_heads / heads_per_group) * dk], v [N, >= n_heads * dv] with row strides (elements);
// log_a, b [N, >= n_heads] with row strides; skip [n_heads] or null; m_tok [N, n_heads] dense or null
// (needed with a normalizer); state [slots][n_heads][dv + normalizer][dk]; o [N, n_heads * dv] dense.
MV_API int mv_scalar_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                          const float* log_a, int ld_a, const float* b, int ld_b, const float* skip,
                          const float* m_tok, float q_scale, float* state, const int* slots, const int* cu, float* o,
                          int n_seqs, int n_heads, int heads_per_group, int dk, int dv, int normalizer,
                          cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || heads_per_group < 1 || n_heads % heads_per_group || (normalizer && !m_tok))
        return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + SS_COLS - 1) / SS_COLS, n_heads, n_seqs);
    const int threads = SS_COLS * SS_PART + (normalizer ? 32 : 0);
    const size_t smem = sizeof(float) * ((size_t)SS_CHUNK * (2 * dk + SS_COLS + 2 + SS_COLS + 1));
#define SS_LAUNCH(R)                                                                                              \
    mv_launch(scalar_scan_kernel<R>, grid, threads, smem, stream, q, ldq, k, ldk, v, ldv, log_a, ld_a, b, ld_b,  \
              skip, m_tok, q_scale, state, slots, cu, o, n_heads, heads_per_group, dk, dv, normalizer)
    if (dk <= 64) SS_LAUNCH(8);
    else if (dk <= 128) SS_LAUNCH(16);
    else SS_LAUNCH(32);
#undef SS_LAUNCH
    return mv_launch_status();
}

// ------------------------------------------------------------------------------------------------
// The log gates of a matrix memory and their running maximum, per sequence and head:
//     i_t = cap tanh((zi_t + bi) / cap),  f_t = log sigmoid(cap tanh((zf_t + bf) / cap)),
//     m_t = max(f_t + m_(t-1), i_t)   (m before a sequence's first token is 0: a zeroed state),
//     log a_t = f_t + m_(t-1) - m_t,  b_t = e^(i_t - m_t).
// A block is one sequence: all threads work out the gates of its tokens, one thread a head then walks the
// maximum (the only part that is sequential), all threads finish b.  m is kept per slot and head.
__device__ __forceinline__ float ss_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

__global__ void __launch_bounds__(256)
memory_gates_kernel(const float* __restrict__ zi, int ld_i, const float* __restrict__ zf, int ld_f,
                    const float* __restrict__ bi, const float* __restrict__ bf, float cap, float* __restrict__ m_state,
                    const int* __restrict__ slots, const int* __restrict__ cu, float* __restrict__ log_a,
                    float* __restrict__ b_out, float* __restrict__ m_tok, int n_heads) {
    mv_pdl_begin();
    const int b = blockIdx.x;
    const int row0 = cu[b], len = cu[b + 1] - row0;
    if (len <= 0) return;
    const float inv_cap = 1.0f / cap;
    for (int idx = threadIdx.x; idx < len * n_heads; idx += blockDim.x) {
        const int t = idx / n_heads, h = idx - t * n_heads;
        const size_t row = (size_t)(row0 + t);
        const float il = cap * tanhf((zi[row * ld_i + h] + bi[h]) * inv_cap);
        const float fl = ss_log_sigmoid(cap * tanhf((zf[row * ld_f + h] + bf[h]) * inv_cap));
        b_out[row * n_heads + h] = il;
        log_a[row * n_heads + h] = fl;
    }
    __syncthreads();
    const int slot = mv_read_slot(slots[b]);
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        float m = m_state[(size_t)slot * n_heads + h];
        for (int t = 0; t < len; ++t) {
            const size_t at = (size_t)(row0 + t) * n_heads + h;
            const float fl = log_a[at], il = b_out[at];
            const float m_new = fmaxf(fl + m, il);
            log_a[at] = fl + m - m_new;
            m_tok[at] = m_new;
            m = m_new;
        }
        if (mv_slot_ok(slots[b])) m_state[(size_t)slot * n_heads + h] = m;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < len * n_heads; idx += blockDim.x) {
        const size_t at = (size_t)row0 * n_heads + idx;
        b_out[at] = expf(b_out[at] - m_tok[at]);
    }
}

// zi, zf: the gates' projections [N, >= n_heads] with row strides; bi, bf [n_heads]; m_state [slots][n_heads];
// log_a, b_out, m_tok [N, n_heads] dense.
MV_API int mv_memory_gates(const float* zi, int ld_i, const float* zf, int ld_f, const float* bi, const float* bf,
                           float cap, float* m_state, const int* slots, const int* cu, float* log_a, float* b_out,
                           float* m_tok, int n_seqs, int n_heads, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!(cap > 0.f) || n_heads < 1) return (int)cudaErrorInvalidValue;
    mv_launch(memory_gates_kernel, n_seqs, 256, 0, stream, zi, ld_i, zf, ld_f, bi, bf, cap, m_state, slots, cu, log_a,
              b_out, m_tok, n_heads);
    return mv_launch_status();
}
