// Linear attention with a per-head decay and a state carried from token to token (the "lightning" mixer):
//
//   q_t = act(q~_t), k_t = act(k~_t) [dim], v_t = act(v~_t) [vdim]      act = silu (or none), float32
//   S_t = lambda_h S_(t-1) + k_t (x) v_t          S [dim, vdim] float32, per (request, head), zero at the start
//   o_t = S_t^T q_t                               float32 [vdim]
//
// A prompt portion of n tokens is taken in chunks of C = 32 tokens.  With S the state before a chunk and i, j
// counting inside it:
//   A_ij = (q_i . k_j) lambda^(i-j)  for j <= i             scores, float32, no softmax
//   o_i  = lambda^(i+1) S^T q_i + sum_(j<=i) A_ij v_j
//   S'   = lambda^n S + sum_j lambda^(n-1-j) k_j (x) v_j     n = tokens of this chunk
// which is the recurrence above written out, so a single decoded token (n = 1) and a portion cut anywhere give the
// same values up to float32 rounding.  Everything is float32 on the CUDA cores: the state, the decay powers, the
// scores and their products with v.
//
// Work split: one block per (sequence, head, slice of 32 value columns): a column of S never meets another
// column, so slices of vdim are independent.  Thread (e, g) = (lane, warp) keeps S[d, e] for d = g, g + 8, ... in
// registers and a copy of the block's S in shared memory for the S^T q products.
//
// A sequence whose state slot is negative or that brings no tokens (the padding of a step laid out for replay) is
// skipped.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int LA_C = 32;        // tokens per chunk
constexpr int LA_WARPS = 8;
constexpr int LA_EV = 32;       // value columns per block

struct LinAttnParams {
    const void* q;              // rows of the packed projection; q, k, v start at these pointers
    const void* k;
    const void* v;
    long long ld;               // row stride of the packed projection, in elements
    float* out;                 // [tokens, heads * vdim] float32
    float* state;               // [slots, heads, dim, vdim] float32
    const float* decay;         // [heads]
    const int* cu_q;            // [seqs + 1]
    const int* state_slots;     // [seqs]
    int heads, dim, vdim, silu;
};

__device__ __forceinline__ float la_act(float x, int silu) { return silu ? __fdividef(x, 1.0f + __expf(-x)) : x; }

template <typename T, int DPT>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_kernel(LinAttnParams p) {
    extern __shared__ float smem[];
    const int D = p.dim, E = p.vdim;
    const int DP = D + 1;
    float* Qs = smem;                      // [C][D + 1]
    float* Ks = Qs + LA_C * DP;            // [C][D + 1]
    float* Vs = Ks + LA_C * DP;            // [C][EV]
    float* As = Vs + LA_C * LA_EV;         // [C][C + 1]
    float* Ss = As + LA_C * (LA_C + 1);    // [D][EV]
    float* pw = Ss + D * LA_EV;            // [C + 1] powers of the decay
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int s = blockIdx.x, h = blockIdx.y, e0 = blockIdx.z * LA_EV;
    const int e = e0 + lane;
    const bool e_ok = e < E;
    const float lam = p.decay[h];
    if (threadIdx.x <= LA_C) pw[threadIdx.x] = powf(lam, (float)threadIdx.x);
    pdl_launch_dependents();
    pdl_wait();
    const int slot = p.state_slots[s];
    const int t_beg = p.cu_q[s], n_tok = p.cu_q[s + 1] - t_beg;
    if (slot < 0 || n_tok <= 0) return;
    float* Sg = p.state + (((size_t)slot * p.heads + h) * D) * E;
    float S[DPT];
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = g + LA_WARPS * r;
        S[r] = (d < D && e_ok) ? Sg[(size_t)d * E + e] : 0.f;
        if (d < D) Ss[d * LA_EV + lane] = S[r];
    }
    const T* qb = static_cast<const T*>(p.q) + (size_t)h * D;
    const T* kb = static_cast<const T*>(p.k) + (size_t)h * D;
    const T* vb = static_cast<const T*>(p.v) + (size_t)h * E;
    constexpr int VN = Vec16<T>::N;
    const bool vec_ok = D % VN == 0 && p.ld % VN == 0 && aligned16(qb) && aligned16(kb);
    for (int c0 = 0; c0 < n_tok; c0 += LA_C) {
        const int n = min(LA_C, n_tok - c0);
        __syncthreads();                    // the chunk before is consumed, Ss and pw are written
        if (vec_ok) {
            // 16 bytes of q and of k per thread and turn
            const int vecs = D / VN;
            for (int idx = threadIdx.x; idx < LA_C * vecs; idx += blockDim.x) {
                const int i = idx / vecs, d = (idx % vecs) * VN;
                float qf[VN], kf[VN];
                if (i < n) {
                    const size_t row = (size_t)(t_beg + c0 + i) * p.ld;
                    Vec16<T> qv, kv;
                    qv.raw = *reinterpret_cast<const decltype(qv.raw)*>(qb + row + d);
                    kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(kb + row + d);
                    qv.unpack(qf);
                    kv.unpack(kf);
#pragma unroll
                    for (int u = 0; u < VN; ++u) {
                        qf[u] = la_act(qf[u], p.silu);
                        kf[u] = la_act(kf[u], p.silu);
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < VN; ++u) qf[u] = kf[u] = 0.f;
                }
#pragma unroll
                for (int u = 0; u < VN; ++u) {
                    Qs[i * DP + d + u] = qf[u];
                    Ks[i * DP + d + u] = kf[u];
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < LA_C * D; idx += blockDim.x) {
                const int i = idx / D, d = idx % D;
                float qv = 0.f, kv = 0.f;
                if (i < n) {
                    const size_t row = (size_t)(t_beg + c0 + i) * p.ld;
                    qv = la_act(to_float(qb[row + d]), p.silu);
                    kv = la_act(to_float(kb[row + d]), p.silu);
                }
                Qs[i * DP + d] = qv;
                Ks[i * DP + d] = kv;
            }
        }
        for (int idx = threadIdx.x; idx < LA_C * LA_EV; idx += blockDim.x) {
            const int i = idx / LA_EV, ee = idx % LA_EV;
            float vv = 0.f;
            if (i < n && e0 + ee < E) vv = la_act(to_float(vb[(size_t)(t_beg + c0 + i) * p.ld + e0 + ee]), p.silu);
            Vs[idx] = vv;
        }
        __syncthreads();
        // scores: warp g takes rows i = g, g + 8, ...; lane j the key
        for (int i = g; i < LA_C; i += LA_WARPS) {
            float a = 0.f;
            if (lane <= i && i < n) {
                const float* qi = Qs + i * DP;
                const float* kj = Ks + lane * DP;
                for (int d = 0; d < D; ++d) a = fmaf(qi[d], kj[d], a);
                a *= pw[i - lane];
            }
            As[i * (LA_C + 1) + lane] = a;
        }
        __syncthreads();
        // outputs: thread (e, g) takes rows i = g, g + 8, g + 16, g + 24
        {
            float acc[LA_C / LA_WARPS];
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = 0.f;
            for (int d = 0; d < D; ++d) {
                const float sv = Ss[d * LA_EV + lane];
#pragma unroll
                for (int r = 0; r < LA_C / LA_WARPS; ++r) acc[r] = fmaf(Qs[(g + LA_WARPS * r) * DP + d], sv, acc[r]);
            }
#pragma unroll
            for (int r = 0; r < LA_C / LA_WARPS; ++r) {
                const int i = g + LA_WARPS * r;
                if (i >= n) continue;
                float o = acc[r] * pw[i + 1];
                for (int j = 0; j <= i; ++j) o = fmaf(As[i * (LA_C + 1) + j], Vs[j * LA_EV + lane], o);
                if (e_ok) p.out[(size_t)(t_beg + c0 + i) * ((size_t)p.heads * E) + (size_t)h * E + e] = o;
            }
        }
        __syncthreads();                    // every reader of Ss is done
        // state: S[d, e] = lambda^n S[d, e] + sum_j lambda^(n-1-j) k_j[d] v_j[e]
        {
            const float keep = pw[n];
            float add[DPT];
#pragma unroll
            for (int r = 0; r < DPT; ++r) add[r] = 0.f;
            for (int j = 0; j < n; ++j) {
                const float vj = Vs[j * LA_EV + lane] * pw[n - 1 - j];
#pragma unroll
                for (int r = 0; r < DPT; ++r) {
                    const int d = g + LA_WARPS * r;
                    if (d < D) add[r] = fmaf(Ks[j * DP + d], vj, add[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < DPT; ++r) {
                const int d = g + LA_WARPS * r;
                S[r] = fmaf(keep, S[r], add[r]);
                if (d < D) Ss[d * LA_EV + lane] = S[r];
            }
        }
    }
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = g + LA_WARPS * r;
        if (d < D && e_ok) Sg[(size_t)d * E + e] = S[r];
    }
}

template <typename T, int DPT>
static int launch_linear_attention(const LinAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(linear_attention_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("linear_attention: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
    }
    LLMK_CHECK_LAUNCH_RC("linear_attention", llmk_launch(linear_attention_kernel<T, DPT>, grid, dim3(LA_WARPS * 32), smem, s, true, p));
    return LLMK_OK;
}

template <typename T>
static int dispatch_linear_attention(const LinAttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    const int dpt = ceil_div(p.dim, LA_WARPS);
    if (dpt <= 4) return launch_linear_attention<T, 4>(p, grid, smem, s);
    if (dpt <= 8) return launch_linear_attention<T, 8>(p, grid, smem, s);
    if (dpt <= 16) return launch_linear_attention<T, 16>(p, grid, smem, s);
    return launch_linear_attention<T, 32>(p, grid, smem, s);
}

// q, k, v: pointers to the first row's q, k and v inside the packed projection (rows `ld` elements apart, heads
// side by side); out float32 [tokens, heads * vdim]; state float32 [slots, heads, dim, vdim]; decay float32 [heads].
LLMK_EXPORT int llmk_linear_attention(float* out, const void* q, const void* k, const void* v, long long ld, float* state,
                                      const float* decay, const int* cu_q, const int* state_slots, int n_seqs, int heads,
                                      int dim, int vdim, int silu, int dtype, void* stream) {
    if (n_seqs <= 0) return LLMK_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0) LLMK_FAIL("linear_attention: bad sizes (heads %d, dim %d, vdim %d)", heads, dim, vdim);
    if (dim > 32 * LA_WARPS) LLMK_FAIL("linear_attention: dim %d is more than %d", dim, 32 * LA_WARPS);
    if (heads > 65535) LLMK_FAIL("linear_attention: too many heads");
    LinAttnParams p;
    p.q = q; p.k = k; p.v = v; p.ld = ld; p.out = out; p.state = state; p.decay = decay; p.cu_q = cu_q;
    p.state_slots = state_slots; p.heads = heads; p.dim = dim; p.vdim = vdim; p.silu = silu;
    const size_t smem = ((size_t)2 * LA_C * (dim + 1) + LA_C * LA_EV + LA_C * (LA_C + 1) + (size_t)dim * LA_EV + LA_C + 1) * sizeof(float);
    dim3 grid(n_seqs, heads, ceil_div(vdim, LA_EV));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == LLMK_F32) return dispatch_linear_attention<float>(p, grid, smem, s);
    if (dtype == LLMK_BF16) return dispatch_linear_attention<bf16>(p, grid, smem, s);
    LLMK_FAIL("linear_attention: unknown dtype %d", dtype);
}
