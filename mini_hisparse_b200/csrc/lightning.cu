// Linear attention with a fixed decay per head ("lightning attention") over a state that is carried
// from step to step:
//
//   q_t = silu(.), k_t = silu(.) [dk], v_t = silu(.) [dv]  of head h, from one stacked product
//   S_t = lambda_h S_(t-1) + k_t v_t^T        S is [dk][dv], float32, one per request slot and head
//   o_t = S_t^T q_t
//
// S is kept as float32 and so is every term of its update and of o: the product's float32 outputs
// (or split-K parts, summed in order) go through silu in float32; on the CUDA-core routes nothing is
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
#include "mma_helpers.cuh"

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
    // one element of the state per thread (blockIdx.z tiles the elements): the walk over the chunks is a
    // chain of dependent sums, but its loads do not depend on it and are asked for eight chunks ahead
    const int idx = blockIdx.z * blockDim.x + threadIdx.x;
    if (idx >= dk * dv) return;
    const int n_full = chunks[4 * c0 + 2];
    const float lam_full = powf(lam, (float)n_full);
    const size_t stride = (size_t)a.H * dk * dv;
    float* u = U + ((size_t)c0 * a.H + h) * dk * dv + idx;
    float S = fresh ? 0.f : slot[idx];
    for (int c = 0; c < nc; c += 8) {
        float own[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) own[i] = c + i < nc ? u[(size_t)(c + i) * stride] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (c + i < nc) {
                u[(size_t)(c + i) * stride] = S;
                const int n = chunks[4 * (c0 + c + i) + 2];
                S = fmaf(n == n_full ? lam_full : powf(lam, (float)n), S, own[i]);
            }
        }
    }
    if (a.writable) slot[idx] = S;
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


// ---- chunked, on the tensor cores (the bfloat16 runtime) ---------------------------------------------------
// The same three steps with mma.sync m16n8k16 (bfloat16 operands, float32 accumulation) for steps (1)
// and (3); step (2) is the kernel above.  q, k and v are rounded to bfloat16 after silu (they are
// activations of projections).  What the recurrence adds up stays at float32's reach: a float32 number
// that must be an operand (a key times its power of lambda, a state, a decayed score) goes in as the sum
// of two bfloat16 numbers, the rounded value and what the rounding lost, with a product for each (16
// bits of mantissa instead of 8); powers of lambda, the masks and all sums are float32.
// Chunks are 64 tokens; DK and DV are the widths padded to 32, 64 or 128 (the tails are zero).
constexpr int TC_C = 64;

__device__ __forceinline__ float load_raw(const LightArgs& a, size_t idx) {
    float v = a.proj[idx];
    for (int s = 1; s < a.nsplit; ++s) v += a.proj[idx + (size_t)s * a.split_stride];
    return v;
}

// N * W values of the chunk's rows [t0, t0 + n) and columns [col0, col0 + w) of the product (zero outside),
// through silu, handed to `put(row, column, value)`: eight loads are asked for before the first is used (a
// thread that waits for every load in turn spends the kernel waiting).
template <int W, int NT, typename Put>
__device__ __forceinline__ void load_tile_silu(const LightArgs& a, int t0, int n, int col0, int w, Put put) {
    constexpr int TOTAL = TC_C * W;
    // four elements a load where rows and columns allow it (16-byte aligned): a quarter of the requests
    const bool vec = (w & 3) == 0 && (col0 & 3) == 0 && (a.ld & 3) == 0 && (a.split_stride & 3) == 0 &&
                     ((uintptr_t)a.proj & 15) == 0;
    if (vec) {
        for (int base = 0; base < TOTAL; base += NT * 4 * 4) {
            float4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + (u * NT + (int)threadIdx.x) * 4;
                const int j = idx / W, e = idx - j * W;
                raw[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < TOTAL && j < n && e < w) {
                    const float* p = a.proj + (size_t)(t0 + j) * a.ld + col0 + e;
                    raw[u] = *(const float4*)p;
                    for (int s = 1; s < a.nsplit; ++s) {
                        const float4 x = *(const float4*)(p + (size_t)s * a.split_stride);
                        raw[u].x += x.x; raw[u].y += x.y; raw[u].z += x.z; raw[u].w += x.w;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + (u * NT + (int)threadIdx.x) * 4;
                const int j = idx / W, e = idx - j * W;
                if (idx < TOTAL) {
                    put(j, e, siluf(raw[u].x)); put(j, e + 1, siluf(raw[u].y));
                    put(j, e + 2, siluf(raw[u].z)); put(j, e + 3, siluf(raw[u].w));
                }
            }
        }
        return;
    }
    for (int base = 0; base < TOTAL; base += NT * 8) {
        float raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = base + u * NT + (int)threadIdx.x;
            const int j = idx / W, e = idx - j * W;
            raw[u] = (idx < TOTAL && j < n && e < w) ? load_raw(a, (size_t)(t0 + j) * a.ld + col0 + e) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = base + u * NT + (int)threadIdx.x;
            const int j = idx / W, e = idx - j * W;
            if (idx < TOTAL) put(j, e, siluf(raw[u]));
        }
    }
}

__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

constexpr int STATE_THREADS = 128;      // four warps load, convert and multiply (eight were slower: 96 against 79 us)
constexpr int OUT_THREADS = 512;        // all load and convert; the first eight warps multiply

template <int DK, int DV>
__global__ void __launch_bounds__(STATE_THREADS)
lightning_chunk_state_tc_kernel(const LightArgs a, const int* __restrict__ chunks, float* __restrict__ U) {
    constexpr int LDK = DK + 8, LDV = DV + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* kh = (__nv_bfloat16*)smem_raw;          // [C][LDK] keys times lambda^(n-1-j), rounded
    __nv_bfloat16* kl = kh + TC_C * LDK;                    // what the rounding lost
    __nv_bfloat16* vs = kl + TC_C * LDK;                    // [C][LDV]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const int dk = a.dk, dv = a.dv;
    const float lam = a.decay[h];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float pw_s[TC_C];                  // lambda^(n-1-j)
    if (tid < TC_C) pw_s[tid] = tid < n ? powf(lam, (float)(n - 1 - tid)) : 0.f;
    __syncthreads();
    // the key as the other kernel sees it (rounded once), times its power of lambda
    load_tile_silu<DK, STATE_THREADS>(a, t0, n, a.k0 + h * dk, dk, [&](int j, int e, float v) {
        split_bf16(__bfloat162float(__float2bfloat16_rn(v)) * pw_s[j], kh[j * LDK + e], kl[j * LDK + e]);
    });
    load_tile_silu<DV, STATE_THREADS>(a, t0, n, a.v0 + h * dv, dv, [&](int j, int e, float v) { vs[j * LDV + e] = __float2bfloat16_rn(v); });
    __syncthreads();
    // U [DK][DV] = K'^T V: warp w owns the rows w * DK/4 ... of U, in tiles of 16
    constexpr int MT = DK / 64;            // 16-row tiles per warp (DK = 32: two warps have none)
    constexpr int MTILES = MT > 0 ? MT : 1;
    const uint32_t kh_s = (uint32_t)__cvta_generic_to_shared(kh), kl_s = (uint32_t)__cvta_generic_to_shared(kl);
    const uint32_t v_s = (uint32_t)__cvta_generic_to_shared(vs);
    if (warp >= 4 || (DK == 32 && warp >= 2)) return;
    float u[MTILES][DV / 8][4];
#pragma unroll
    for (int m = 0; m < MTILES; ++m)
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) u[m][i][0] = u[m][i][1] = u[m][i][2] = u[m][i][3] = 0.f;
    const int row0 = DK == 32 ? warp * 16 : warp * (DK / 4);
#pragma unroll
    for (int ks = 0; ks < TC_C / 16; ++ks) {
        uint32_t ah[MTILES][4], al[MTILES][4];
#pragma unroll
        for (int m = 0; m < MTILES; ++m) {
            const int r = ks * 16 + (lane & 7) + 8 * (lane >> 4), cc = row0 + m * 16 + 8 * ((lane >> 3) & 1);
            ldmatrix_x4_trans(kh_s + (r * LDK + cc) * 2, ah[m][0], ah[m][1], ah[m][2], ah[m][3]);
            ldmatrix_x4_trans(kl_s + (r * LDK + cc) * 2, al[m][0], al[m][1], al[m][2], al[m][3]);
        }
#pragma unroll
        for (int i = 0; i < DV / 8; i += 2) {
            uint32_t b0, b1, b2, b3;
            const int r = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = i * 8 + 8 * (lane >> 4);
            ldmatrix_x4_trans(v_s + (r * LDV + cc) * 2, b0, b1, b2, b3);
#pragma unroll
            for (int m = 0; m < MTILES; ++m) {
                mma_bf16(u[m][i], ah[m], b0, b1);
                mma_bf16(u[m][i + 1], ah[m], b2, b3);
                mma_bf16(u[m][i], al[m], b0, b1);
                mma_bf16(u[m][i + 1], al[m], b2, b3);
            }
        }
    }
    float* dst = U + ((size_t)c * a.H + h) * dk * dv;
#pragma unroll
    for (int m = 0; m < MTILES; ++m)
#pragma unroll
        for (int i = 0; i < DV / 8; ++i)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int r = row0 + m * 16 + (lane >> 2) + 8 * (x >> 1), e = i * 8 + (lane & 3) * 2 + (x & 1);
                if (r < dk && e < dv) dst[r * dv + e] = u[m][i][x];
            }
}

// `staged`: the launch brought room for the chunk's raw float32 tiles: they are copied to shared memory by
// cp.async, all requests in flight at once (one memory latency instead of one per batch of loads; with one
// CTA of four warps per SM nothing else hides it), and converted from there.  Needs 16-byte aligned rows
// and a product that is not split.
template <int DK, int DV>
__global__ void __launch_bounds__(OUT_THREADS)
lightning_chunk_out_tc_kernel(const LightArgs a, const int* __restrict__ chunks, const float* __restrict__ U, int staged) {
    constexpr int LDK = DK + 8, LDV = DV + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;          // [C][LDK]
    __nv_bfloat16* ks = qs + TC_C * LDK;                    // [C][LDK]
    __nv_bfloat16* vs = ks + TC_C * LDK;                    // [C][LDV]
    __nv_bfloat16* sh = vs + TC_C * LDV;                    // [DK][LDV] the state before the chunk, rounded
    __nv_bfloat16* sl = sh + DK * LDV;                      // what the rounding lost
    float* pw = (float*)(sl + DK * LDV);                    // [C + 1] powers of lambda
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y;
    const int t0 = chunks[4 * c + 1], n = chunks[4 * c + 2];
    const int dk = a.dk, dv = a.dv;
    const float lam = a.decay[h];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* S = U + ((size_t)c * a.H + h) * dk * dv;
    for (int i = tid; i <= TC_C; i += OUT_THREADS) pw[i] = powf(lam, (float)i);
    if (staged) {
        float* stage = pw + ((TC_C + 1 + 3) & ~3);                 // 16-byte aligned behind the powers
        const uint32_t stage_s = (uint32_t)__cvta_generic_to_shared(stage);
        auto issue = [&](int W, int col0, int w, int at) {
            for (int idx = tid * 4; idx < TC_C * W; idx += OUT_THREADS * 4) {
                const int j = idx / W, e = idx - j * W;
                const bool live = j < n && e < w;
                const float* src = live ? a.proj + (size_t)(t0 + j) * a.ld + col0 + e : a.proj;
                cp_async16(stage_s + (at + idx) * 4, src, live ? 16 : 0);
            }
        };
        issue(DK, a.q0 + h * dk, dk, 0);
        issue(DK, a.k0 + h * dk, dk, TC_C * DK);
        issue(DV, a.v0 + h * dv, dv, 2 * TC_C * DK);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        for (int idx = tid; idx < TC_C * DK; idx += OUT_THREADS) {
            const int j = idx / DK, e = idx - j * DK;
            qs[j * LDK + e] = __float2bfloat16_rn(siluf(stage[idx]));
            ks[j * LDK + e] = __float2bfloat16_rn(siluf(stage[TC_C * DK + idx]));
        }
        for (int idx = tid; idx < TC_C * DV; idx += OUT_THREADS) {
            const int j = idx / DV, e = idx - j * DV;
            vs[j * LDV + e] = __float2bfloat16_rn(siluf(stage[2 * TC_C * DK + idx]));
        }
        __syncthreads();                                            // the staging room is used again
        for (int idx = tid * 4; idx < DK * DV; idx += OUT_THREADS * 4) {
            const int r = idx / DV, e = idx - r * DV;
            const bool live = r < dk && e < dv;
            cp_async16(stage_s + idx * 4, live ? S + r * dv + e : S, live ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        for (int idx = tid; idx < DK * DV; idx += OUT_THREADS) {
            const int r = idx / DV, e = idx - r * DV;
            split_bf16(stage[idx], sh[r * LDV + e], sl[r * LDV + e]);
        }
    } else {
    load_tile_silu<DK, OUT_THREADS>(a, t0, n, a.q0 + h * dk, dk, [&](int j, int e, float v) { qs[j * LDK + e] = __float2bfloat16_rn(v); });
    load_tile_silu<DK, OUT_THREADS>(a, t0, n, a.k0 + h * dk, dk, [&](int j, int e, float v) { ks[j * LDK + e] = __float2bfloat16_rn(v); });
    load_tile_silu<DV, OUT_THREADS>(a, t0, n, a.v0 + h * dv, dv, [&](int j, int e, float v) { vs[j * LDV + e] = __float2bfloat16_rn(v); });
    if ((dv & 3) == 0 && (((uintptr_t)S) & 15) == 0) {
        for (int base = 0; base < DK * DV; base += OUT_THREADS * 4 * 4) {
            float4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + (u * OUT_THREADS + tid) * 4;
                const int r = idx / DV, e = idx - r * DV;
                raw[u] = (idx < DK * DV && r < dk && e < dv) ? *(const float4*)(S + r * dv + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + (u * OUT_THREADS + tid) * 4;
                const int r = idx / DV, e = idx - r * DV;
                if (idx < DK * DV) {
                    split_bf16(raw[u].x, sh[r * LDV + e], sl[r * LDV + e]);
                    split_bf16(raw[u].y, sh[r * LDV + e + 1], sl[r * LDV + e + 1]);
                    split_bf16(raw[u].z, sh[r * LDV + e + 2], sl[r * LDV + e + 2]);
                    split_bf16(raw[u].w, sh[r * LDV + e + 3], sl[r * LDV + e + 3]);
                }
            }
        }
    } else {
        for (int base = 0; base < DK * DV; base += OUT_THREADS * 8) {
            float raw[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * OUT_THREADS + tid;
                const int r = idx / DV, e = idx - r * DV;
                raw[u] = (idx < DK * DV && r < dk && e < dv) ? S[r * dv + e] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * OUT_THREADS + tid;
                const int r = idx / DV, e = idx - r * DV;
                if (idx < DK * DV) split_bf16(raw[u], sh[r * LDV + e], sl[r * LDV + e]);
            }
        }
    }
    }
    __syncthreads();
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(qs), k_s = (uint32_t)__cvta_generic_to_shared(ks);
    const uint32_t v_s = (uint32_t)__cvta_generic_to_shared(vs);
    const uint32_t sh_s = (uint32_t)__cvta_generic_to_shared(sh), sl_s = (uint32_t)__cvta_generic_to_shared(sl);
    if (warp >= 8) return;
    const int wrow = (warp & 3) * 16;           // this warp's 16 tokens of the chunk ...
    if (wrow >= n) return;
    constexpr int KSTEPS = DK / 16, DTILES = DV / 16;     // ... and its half of the value columns
    const int col0 = (warp >> 2) * (DV / 2);
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
        const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), cc = k * 16 + 8 * (lane >> 4);
        ldmatrix_x4(q_s + (r * LDK + cc) * 2, qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
    }
    // what the state before the chunk gives: o = lambda^(i+1) (q_i^T S)
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
        for (int i = 0; i < DTILES; i += 2) {
            uint32_t b0, b1, b2, b3;
            const int r = k * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = col0 + i * 8 + 8 * (lane >> 4);
            ldmatrix_x4_trans(sh_s + (r * LDV + cc) * 2, b0, b1, b2, b3);
            mma_bf16(o[i], qf[k], b0, b1);
            mma_bf16(o[i + 1], qf[k], b2, b3);
            ldmatrix_x4_trans(sl_s + (r * LDV + cc) * 2, b0, b1, b2, b3);
            mma_bf16(o[i], qf[k], b0, b1);
            mma_bf16(o[i + 1], qf[k], b2, b3);
        }
    }
    const int ra = wrow + (lane >> 2), rb = ra + 8;          // this thread's two rows
    {
        const float fa = pw[ra + 1], fb = pw[rb + 1];
#pragma unroll
        for (int i = 0; i < DTILES; ++i) { o[i][0] *= fa; o[i][1] *= fa; o[i][2] *= fb; o[i][3] *= fb; }
    }
    // the chunk's own tokens: scores against the keys up to this warp's last row, decayed, times the values
#pragma unroll
    for (int kb = 0; kb < TC_C / 16; ++kb) {          // 16 keys at a time
        if (kb * 16 > wrow + 15) break;                 // keys after the warp's rows: masked anyway
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KSTEPS; k += 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t b0, b1, b2, b3;
                const int r = kb * 16 + j * 8 + (lane & 7), cc = k * 16 + 8 * (lane >> 3);
                ldmatrix_x4(k_s + (r * LDK + cc) * 2, b0, b1, b2, b3);
                mma_bf16(s[j], qf[k], b0, b1);
                mma_bf16(s[j], qf[k + 1], b2, b3);
            }
        }
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float p[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int row = x < 2 ? ra : rb;
                const int col = kb * 16 + j * 8 + (lane & 3) * 2 + (x & 1);
                p[x] = col <= row ? s[j][x] * pw[row - col] : 0.f;
            }
            __nv_bfloat16 hi[4], lo[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) split_bf16(p[x], hi[x], lo[x]);
            ph[j * 2 + 0] = (uint32_t)__bfloat16_as_ushort(hi[0]) | ((uint32_t)__bfloat16_as_ushort(hi[1]) << 16);
            ph[j * 2 + 1] = (uint32_t)__bfloat16_as_ushort(hi[2]) | ((uint32_t)__bfloat16_as_ushort(hi[3]) << 16);
            pl[j * 2 + 0] = (uint32_t)__bfloat16_as_ushort(lo[0]) | ((uint32_t)__bfloat16_as_ushort(lo[1]) << 16);
            pl[j * 2 + 1] = (uint32_t)__bfloat16_as_ushort(lo[2]) | ((uint32_t)__bfloat16_as_ushort(lo[3]) << 16);
        }
#pragma unroll
        for (int i = 0; i < DTILES; i += 2) {
            uint32_t b0, b1, b2, b3;
            const int r = kb * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = col0 + i * 8 + 8 * (lane >> 4);
            ldmatrix_x4_trans(v_s + (r * LDV + cc) * 2, b0, b1, b2, b3);
            mma_bf16(o[i], ph, b0, b1);
            mma_bf16(o[i + 1], ph, b2, b3);
            mma_bf16(o[i], pl, b0, b1);
            mma_bf16(o[i + 1], pl, b2, b3);
        }
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int row = x < 2 ? ra : rb, e = col0 + i * 8 + (lane & 3) * 2 + (x & 1);
            if (row < n && e < dv) a.out[(size_t)(t0 + row) * a.H * dv + h * dv + e] = o[i][x];
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
    launch_kernel(lightning_chunk_prefix_kernel, dim3(num_segs, H, (dk * dv + 255) / 256), dim3(256), 0, stream, a, seg_chunks, chunks, U);
    if (check_launch("lightning_chunk_prefix")) return -1;
    launch_kernel(lightning_chunk_out_kernel, dim3(num_chunks, H), dim3(256), s3, stream, a, chunks, (const float*)U, C);
    return check_launch("lightning_chunk_out");
}

namespace {
template <int DK, int DV>
int launch_chunked_tc(const LightArgs& a, const int* chunks, int num_chunks, const int* seg_chunks, int num_segs,
                      float* U, cudaStream_t stream) {
    constexpr size_t s1 = 2 * ((size_t)2 * TC_C * (DK + 8) + (size_t)TC_C * (DV + 8));
    constexpr size_t s3 = 2 * ((size_t)2 * TC_C * (DK + 8) + (size_t)TC_C * (DV + 8) + (size_t)2 * DK * (DV + 8)) + 4 * (TC_C + 1);
    if (allow_smem(lightning_chunk_state_tc_kernel<DK, DV>, s1, "lightning_chunk_state_tc")) return -1;
    // room for the raw tiles of the staged route, if an SM has it and rows are 16-byte aligned
    constexpr size_t stage_floats = (size_t)TC_C * (2 * DK + DV) > (size_t)DK * DV ? (size_t)TC_C * (2 * DK + DV) : (size_t)DK * DV;
    constexpr size_t s3_staged = s3 + 16 + 4 * stage_floats;
    const bool staged = s3_staged <= 227 * 1024 && a.nsplit == 1 && (a.dk & 3) == 0 && (a.dv & 3) == 0 && (a.ld & 3) == 0 &&
                        (a.q0 & 3) == 0 && (a.k0 & 3) == 0 && (a.v0 & 3) == 0 && ((uintptr_t)a.proj & 15) == 0 &&
                        ((uintptr_t)U & 15) == 0;
    const size_t s3_used = staged ? s3_staged : s3;
    if (allow_smem(lightning_chunk_out_tc_kernel<DK, DV>, s3_used, "lightning_chunk_out_tc")) return -1;
    launch_kernel(lightning_chunk_state_tc_kernel<DK, DV>, dim3(num_chunks, a.H), dim3(STATE_THREADS), s1, stream, a, chunks, U);
    if (check_launch("lightning_chunk_state_tc")) return -1;
    launch_kernel(lightning_chunk_prefix_kernel, dim3(num_segs, a.H, (a.dk * a.dv + 255) / 256), dim3(256), 0, stream, a, seg_chunks, chunks, U);
    if (check_launch("lightning_chunk_prefix")) return -1;
    launch_kernel(lightning_chunk_out_tc_kernel<DK, DV>, dim3(num_chunks, a.H), dim3(OUT_THREADS), s3_used, stream, a, chunks,
                  (const float*)U, staged ? 1 : 0);
    return check_launch("lightning_chunk_out_tc");
}
template <int DK>
int dispatch_tc_dv(int dvp, const LightArgs& a, const int* chunks, int num_chunks, const int* seg_chunks, int num_segs,
                   float* U, cudaStream_t stream) {
    switch (dvp) {
        case 32: return launch_chunked_tc<DK, 32>(a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
        case 64: return launch_chunked_tc<DK, 64>(a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
        case 128: return launch_chunked_tc<DK, 128>(a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
    }
    return fail("lightning_chunked_tc: values %d wide", dvp);
}
int pad_width(int d) { return d <= 32 ? 32 : d <= 64 ? 64 : 128; }
}  // namespace

MHB_EXPORT int mhb_lightning_chunked_tc_supports(int dk, int dv) { return dk >= 1 && dk <= 128 && dv >= 1 && dv <= 128; }

// The chunked route on the tensor cores; chunks of exactly 64 tokens (the last of a segment may be shorter).
MHB_EXPORT int mhb_lightning_chunked_tc(const float* proj, int nsplit, long long split_stride, int ld, int q0, int k0,
                                        int v0, const float* decay, float* state, float* out, const int* tok_seg,
                                        const int* seg_slot, const int* positions, int T, int H, int dk, int dv,
                                        int writable, const int* chunks, int num_chunks, const int* seg_chunks,
                                        int num_segs, float* U, cudaStream_t stream) {
    if (num_chunks <= 0 || num_segs <= 0) return 0;
    if (H > 65535) return fail("lightning: too many heads");
    if (!mhb_lightning_chunked_tc_supports(dk, dv)) return fail("lightning_chunked_tc: widths %d and %d (up to 128)", dk, dv);
    const LightArgs a = make_args(proj, nsplit, split_stride, ld, q0, k0, v0, decay, state, out, tok_seg, seg_slot,
                                  positions, T, H, dk, dv, writable);
    switch (pad_width(dk)) {
        case 32: return dispatch_tc_dv<32>(pad_width(dv), a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
        case 64: return dispatch_tc_dv<64>(pad_width(dv), a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
        default: return dispatch_tc_dv<128>(pad_width(dv), a, chunks, num_chunks, seg_chunks, num_segs, U, stream);
    }
}
