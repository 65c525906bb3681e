// Linear attention with a fixed decay per head ("lightning attention") over a state that is carried
// from step to step:
//
//   q_t = silu(.), k_t = silu(.) [dk], v_t = silu(.) [dv]  of head h, from one stacked product
//   S_t = lambda_h S_(t-1) + k_t v_t^T        S is [dk][dv], float32, one per request slot and head
//   o_t = S_t^T q_t
//
// The state lives in float32 and everything that enters the recurrence is float32: the product's
// float32 outputs (or split-K parts, summed in order) go through silu in float32; nothing is
// rounded to a shorter type before it is added into S or o.
//
// Two routes give the same numbers up to float32 rounding:
//   scan     one CTA per (segment, head) walks the segment's tokens one by one: decoded tokens and
//            short portions
//   chunked  for long portions: (1) every chunk of C tokens builds its own contribution
//            U_c = sum_j lambda^(C-1-j) k_j v_j^T in parallel, (2) one CTA per (segment, head) turns
//            them into the states at the chunks' starts, S_c = lambda^C S_(c-1) + U_(c-1), and leaves
//            the segment's last state in the slot, (3) every chunk computes
//            o_i = lambda^(i+1) S_c^T q_i + sum_(j<=i) lambda^(i-j) (q_i . k_j) v_j  in parallel.
//            Powers of lambda are only ever taken with non-negative exponents, so nothing overflows
//            however small lambda is.
//
// A segment is a run of consecutive tokens of one request in the batch; tok_seg[t] (ascending) names
// the segment of token t and seg_slot[s] its state slot.  A segment whose first token sits at position
// 0 starts from a zero state whatever the slot holds.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

struct LightArgs {
    const float* proj;        // [nsplit][T][ld]: q at column q0, k at k0, v at v0, heads side by side
    int nsplit;
    size_t split_stride;
    int ld, q0, k0, v0;
    const float* decay;       // [H]
    float* state;             // [slots][H][dk][dv]
    float* out;               // [T][H * dv]
    const int* tok_seg;       // [T]
    const int* seg_slot;      // [S]
    const int* positions;     // [T]
    int T, H, dk, dv, writable;
};

__device__ __forceinline__ float siluf(float z) { return z / (1.f + expf(-z)); }

__device__ __forceinline__ float load_silu(const LightArgs& a, size_t idx) {
    float v = a.proj[idx];
    for (int s = 1; s < a.nsplit; ++s) v += a.proj[idx + (size_t)s * a.split_stride];
    return siluf(v);
}

// first token of segment `seg` and one past its last, by bisection of the ascending tok_seg
__device__ __forceinline__ void segment_range(const int* tok_seg, int T, int seg, int& begin, int& end) {
    int lo = 0, hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] < seg) lo = mid + 1; else hi = mid; }
    begin = lo;
    hi = T;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (tok_seg[mid] <= seg) lo = mid + 1; else hi = mid; }
    end = lo;
}

// ---- token by token ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
lightning_scan_kernel(const LightArgs a, int max_tokens) {
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv;
    float* St = sm;                     // [dk][dv]
    float* qs = St + dk * dv;           // [dk]
    float* ks = qs + dk;                // [dk]
    float* vs = ks + dk;                // [dv]
    const int R = max(1, (int)blockDim.x / dv);
    float* po = vs + dv;                // [R][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.x, h = blockIdx.y;
    int t0, t1;
    segment_range(a.tok_seg, a.T, seg, t0, t1);
    if (t1 <= t0 || (max_tokens > 0 && t1 - t0 > max_tokens)) return;      // longer segments go the chunked way
    const float lam = a.decay[h];
    float* slot = a.state + ((size_t)a.seg_slot[seg] * a.H + h) * dk * dv;
    const bool fresh = a.positions[t0] == 0;
    for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) St[i] = fresh ? 0.f : slot[i];
    for (int t = t0; t < t1; ++t) {
        const size_t base = (size_t)t * a.ld;
        for (int i = threadIdx.x; i < 2 * dk + dv; i += blockDim.x) {
            if (i < dk) qs[i] = load_silu(a, base + a.q0 + h * dk + i);
            else if (i < 2 * dk) ks[i - dk] = load_silu(a, base + a.k0 + h * dk + (i - dk));
            else vs[i - 2 * dk] = load_silu(a, base + a.v0 + h * dv + (i - 2 * dk));
        }
        __syncthreads();
        for (int u = threadIdx.x; u < R * dv; u += blockDim.x) {
            const int r = u / dv, j = u - r * dv;
            const float vj = vs[j];
            float part = 0.f;
            for (int i = r; i < dk; i += R) {
                const float s = fmaf(lam, St[i * dv + j], ks[i] * vj);
                St[i * dv + j] = s;
                part = fmaf(s, qs[i], part);
            }
            po[u] = part;
        }
        __syncthreads();
        for (int j = threadIdx.x; j < dv; j += blockDim.x) {
            float o = 0.f;
            for (int r = 0; r < R; ++r) o += po[r * dv + j];
            a.out[(size_t)t * a.H * dv + h * dv + j] = o;
        }
    }
    __syncthreads();
    if (a.writable)
        for (int i = threadIdx.x; i < dk * dv; i += blockDim.x) slot[i] = St[i];
}

// ---- chunked: (1) every chunk's own contribution -----------------------------------------------------
// work item c of the list: {segment, first token, tokens (<= C), index of the chunk in its segment};
// U[c][h] = sum_j lambda^(n-1-j) k_j v_j^T
__global__ void __launch_bounds__(256)
lightning_chunk_state_kernel(const LightArgs a, const int* __restrict__ chunks, float* __restrict__ U, int C) {
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv;
    float* ks = sm;                     // [C][dk], scaled by lambda^(n-1-j)
    float* vs = ks + C * dk;            // [C][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const float lam = a.decay[h];
    for (int idx = threadIdx.x; idx < n * (dk + dv); idx += blockDim.x) {
        const int j = idx / (dk + dv), e = idx - j * (dk + dv);
        const size_t base = (size_t)(t0 + j) * a.ld;
        if (e < dk) ks[j * dk + e] = load_silu(a, base + a.k0 + h * dk + e) * powf(lam, (float)(n - 1 - j));
        else vs[j * dv + (e - dk)] = load_silu(a, base + a.v0 + h * dv + (e - dk));
    }
    __syncthreads();
    float* u = U + ((size_t)c * a.H + h) * dk * dv;
    for (int idx = threadIdx.x; idx < dk * dv; idx += blockDim.x) {
        const int i = idx / dv, e = idx - i * dv;
        float s = 0.f;
        for (int j = 0; j < n; ++j) s = fmaf(ks[j * dk + i], vs[j * dv + e], s);
        u[idx] = s;
    }
}

// ---- chunked: (2) states at the chunks' starts ---------------------------------------------------------
// One CTA per (listed segment, head): U[c] is replaced by the state BEFORE chunk c, and the state after
// the segment's last chunk goes to the slot.  seg_chunks: {segment, first chunk, chunks, first token}.
__global__ void __launch_bounds__(256)
lightning_chunk_prefix_kernel(const LightArgs a, const int* __restrict__ seg_chunks, const int* __restrict__ chunks,
                              float* __restrict__ U) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int seg = seg_chunks[4 * s], c0 = seg_chunks[4 * s + 1], nc = seg_chunks[4 * s + 2], t0 = seg_chunks[4 * s + 3];
    const int dk = a.dk, dv = a.dv;
    const float lam = a.decay[h];
    float* slot = a.state + ((size_t)a.seg_slot[seg] * a.H + h) * dk * dv;
    const bool fresh = a.positions[t0] == 0;
    for (int idx = threadIdx.x; idx < dk * dv; idx += blockDim.x) {
        float S = fresh ? 0.f : slot[idx];
        for (int c = c0; c < c0 + nc; ++c) {
            float* u = U + ((size_t)c * a.H + h) * dk * dv + idx;
            const float own = *u;
            *u = S;
            S = fmaf(powf(lam, (float)chunks[4 * c + 2]), S, own);
        }
        if (a.writable) slot[idx] = S;
    }
}

// ---- chunked: (3) outputs -----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
lightning_chunk_out_kernel(const LightArgs a, const int* __restrict__ chunks, const float* __restrict__ U, int C) {
    extern __shared__ float sm[];
    const int dk = a.dk, dv = a.dv;
    float* qs = sm;                     // [C][dk + 1]
    float* ks = qs + C * (dk + 1);      // [C][dk + 1]
    float* vs = ks + C * (dk + 1);      // [C][dv]
    float* A = vs + C * dv;             // [C][C + 1] decayed scores
    float* pw = A + C * (C + 1);        // [C + 1] powers of lambda
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const float lam = a.decay[h];
    for (int idx = threadIdx.x; idx < n * (2 * dk + dv); idx += blockDim.x) {
        const int j = idx / (2 * dk + dv), e = idx - j * (2 * dk + dv);
        const size_t base = (size_t)(t0 + j) * a.ld;
        if (e < dk) qs[j * (dk + 1) + e] = load_silu(a, base + a.q0 + h * dk + e);
        else if (e < 2 * dk) ks[j * (dk + 1) + (e - dk)] = load_silu(a, base + a.k0 + h * dk + (e - dk));
        else vs[j * dv + (e - 2 * dk)] = load_silu(a, base + a.v0 + h * dv + (e - 2 * dk));
    }
    for (int i = threadIdx.x; i <= C; i += blockDim.x) pw[i] = powf(lam, (float)i);
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * n; idx += blockDim.x) {
        const int i = idx / n, j = idx - i * n;
        float s = 0.f;
        if (j <= i) {
            const float* qi = qs + i * (dk + 1);
            const float* kj = ks + j * (dk + 1);
            for (int e = 0; e < dk; ++e) s = fmaf(qi[e], kj[e], s);
            s *= pw[i - j];
        }
        A[i * (C + 1) + j] = s;
    }
    __syncthreads();
    const float* S = U + ((size_t)c * a.H + h) * dk * dv;
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int i = idx / dv, e = idx - i * dv;
        float inter = 0.f;
        const float* qi = qs + i * (dk + 1);
        for (int r = 0; r < dk; ++r) inter = fmaf(S[r * dv + e], qi[r], inter);
        float o = inter * pw[i + 1];
        const float* Ai = A + i * (C + 1);
        for (int j = 0; j <= i; ++j) o = fmaf(Ai[j], vs[j * dv + e], o);
        a.out[(size_t)(t0 + i) * a.H * dv + h * dv + e] = o;
    }
}

template <typename Kern>
int allow_smem(Kern kern, size_t smem, const char* what) {
    if (smem > 227 * 1024) return fail("%s: %zu bytes of shared memory are more than an SM has", what, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("%s: shared memory %zu: %s", what, smem, cudaGetErrorString(e));
    }
    return 0;
}

LightArgs make_args(const float* proj, int nsplit, long long split_stride, int ld, int q0, int k0, int v0,
                    const float* decay, float* state, float* out, const int* tok_seg, const int* seg_slot,
                    const int* positions, int T, int H, int dk, int dv, int writable) {
    LightArgs a;
    a.proj = proj; a.nsplit = nsplit; a.split_stride = (size_t)split_stride; a.ld = ld; a.q0 = q0; a.k0 = k0;
    a.v0 = v0; a.decay = decay; a.state = state; a.out = out; a.tok_seg = tok_seg; a.seg_slot = seg_slot;
    a.positions = positions; a.T = T; a.H = H; a.dk = dk; a.dv = dv; a.writable = writable;
    return a;
}
}  // namespace

// Every segment of at most max_tokens tokens (0: every segment), token by token.
MHB_EXPORT int mhb_lightning_scan(const float* proj, int nsplit, long long split_stride, int ld, int q0, int k0,
                                  int v0, const float* decay, float* state, float* out, const int* tok_seg,
                                  const int* seg_slot, const int* positions, int T, int S, int H, int dk, int dv,
                                  int writable, int max_tokens, cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    if (H > 65535) return fail("lightning: too many heads");
    const LightArgs a = make_args(proj, nsplit, split_stride, ld, q0, k0, v0, decay, state, out, tok_seg, seg_slot,
                                  positions, T, H, dk, dv, writable);
    const int R = 256 / dv > 1 ? 256 / dv : 1;
    const size_t smem = sizeof(float) * ((size_t)dk * dv + 2 * dk + dv + (size_t)R * dv);
    if (allow_smem(lightning_scan_kernel, smem, "lightning_scan")) return -1;
    launch_kernel(lightning_scan_kernel, dim3(S, H), dim3(256), smem, stream, a, max_tokens);
    return check_launch("lightning_scan");
}

// Shared memory of the chunked route for chunks of C tokens (the host picks the largest C that fits).
MHB_EXPORT long long mhb_lightning_chunk_smem(int dk, int dv, int C) {
    const size_t s1 = sizeof(float) * ((size_t)C * (dk + dv));
    const size_t s3 = sizeof(float) * ((size_t)2 * C * (dk + 1) + (size_t)C * dv + (size_t)C * (C + 1) + C + 1);
    return (long long)(s1 > s3 ? s1 : s3);
}

// The listed chunks (4 ints each) of the listed segments (4 ints each); U holds num_chunks * H * dk * dv floats.
MHB_EXPORT int mhb_lightning_chunked(const float* proj, int nsplit, long long split_stride, int ld, int q0, int k0,
                                     int v0, const float* decay, float* state, float* out, const int* tok_seg,
                                     const int* seg_slot, const int* positions, int T, int H, int dk, int dv,
                                     int writable, const int* chunks, int num_chunks, const int* seg_chunks,
                                     int num_segs, float* U, int C, cudaStream_t stream) {
    if (num_chunks <= 0 || num_segs <= 0) return 0;
    if (H > 65535) return fail("lightning: too many heads");
    const LightArgs a = make_args(proj, nsplit, split_stride, ld, q0, k0, v0, decay, state, out, tok_seg, seg_slot,
                                  positions, T, H, dk, dv, writable);
    const size_t s1 = sizeof(float) * ((size_t)C * (dk + dv));
    const size_t s3 = sizeof(float) * ((size_t)2 * C * (dk + 1) + (size_t)C * dv + (size_t)C * (C + 1) + C + 1);
    if (allow_smem(lightning_chunk_state_kernel, s1, "lightning_chunk_state")) return -1;
    if (allow_smem(lightning_chunk_out_kernel, s3, "lightning_chunk_out")) return -1;
    launch_kernel(lightning_chunk_state_kernel, dim3(num_chunks, H), dim3(256), s1, stream, a, chunks, U, C);
    if (check_launch("lightning_chunk_state")) return -1;
    launch_kernel(lightning_chunk_prefix_kernel, dim3(num_segs, H), dim3(256), 0, stream, a, seg_chunks, chunks, U);
    if (check_launch("lightning_chunk_prefix")) return -1;
    launch_kernel(lightning_chunk_out_kernel, dim3(num_chunks, H), dim3(256), s3, stream, a, chunks, (const float*)U, C);
    return check_launch("lightning_chunk_out");
}
