// Gated linear attention: a recurrent mixer whose memory per head is a matrix S [key channels, value channels] in
// float32, decayed per key channel and updated by an outer product at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,      a_t = sigmoid(z_t)^(1/tau)
//
// The state row of a sequence lives in the cache's fixed-size state table ([slots, heads * dk * dv]) and is carried
// from step to step; one kernel serves a whole prompt, a portion of one and a single token (it walks the new tokens of
// its sequence in order).  Everything that enters the recurrence besides the projections q, k, v is float32: the decay
// logits z arrive in float32, a = exp(-softplus(-z) / tau) is formed here, the state and the sums stay float32.
//
//  * gla_scan: a block owns 32 value columns of one head of one sequence; a thread owns one column and every fourth
//    key channel of it (KPT state values in registers); q, k, a and v of eight tokens at a time are staged in shared
//    memory; o_t is completed by two shuffles.
//  * gla_out: per (token, head) one warp: RMS norm of o over the value channels with a weight shared by the heads,
//    times silu of the output gate.
#include "common.cuh"

constexpr int GLA_KS = 4;         // key-channel slices (lanes that share a value column)
constexpr int GLA_COLS = 32;      // value columns of a block
constexpr int GLA_THREADS = GLA_KS * GLA_COLS;
constexpr int GLA_CHUNK = 8;      // tokens staged at a time

struct GlaParams {
    const void* q;            // packed projections [T, row_stride]: head h's queries at q + h * dk
    const void* k;            // the same buffer at its first key column
    const void* v;            // the same buffer at its first value column
    int row_stride;
    const float* z;           // decay logits [T, z_stride], head h at h * dk
    int z_stride;
    float* state;             // [slots, H * dk * dv]
    const int* seq_start;     // [B + 1]
    const int* seq_slot;      // [B]
    float* out;               // [T, H * dv]
    int H, dk, dv;
    float q_scale, inv_tau;
};

template <typename T, int KPT>
__global__ void __launch_bounds__(GLA_THREADS) gla_scan_kernel(GlaParams p) {
    extern __shared__ float sm[];
    constexpr int DKP = GLA_KS * KPT;                 // key channels, padded
    float* sq = sm;                                   // [CHUNK][DKP]
    float* sk = sq + GLA_CHUNK * DKP;
    float* sa = sk + GLA_CHUNK * DKP;
    float* sv = sa + GLA_CHUNK * DKP;                 // [CHUNK][COLS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane & (GLA_KS - 1), jl = lane / GLA_KS;
    const int cloc = warp * (32 / GLA_KS) + jl;       // column within the block
    const int col = blockIdx.x * GLA_COLS + cloc;
    const int h = blockIdx.y, b = blockIdx.z;
    const int dk = p.dk, dv = p.dv;
    llb_grid_dependency_sync();
    const int tok0 = p.seq_start[b], n = p.seq_start[b + 1] - tok0;
    float* st = p.state + ((size_t)p.seq_slot[b] * p.H + h) * dk * dv;
    float S[KPT];
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
        int i = part + GLA_KS * m;
        S[m] = (i < dk && col < dv) ? st[(size_t)i * dv + col] : 0.f;
    }
    const T* qb = (const T*)p.q;
    const T* kb = (const T*)p.k;
    const T* vb = (const T*)p.v;
    for (int c0 = 0; c0 < n; c0 += GLA_CHUNK) {
        const int nc = min(GLA_CHUNK, n - c0);
        __syncthreads();
        for (int idx = tid; idx < nc * DKP; idx += GLA_THREADS) {
            int t = idx / DKP, i = idx - t * DKP;
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (i < dk) {
                size_t row = (size_t)(tok0 + c0 + t);
                qv = to_f32(qb[row * p.row_stride + h * dk + i]) * p.q_scale;
                kv = to_f32(kb[row * p.row_stride + h * dk + i]);
                float zz = p.z[row * p.z_stride + h * dk + i];
                // log sigmoid(z) = -softplus(-z) = -(max(-z, 0) + log(1 + e^-|z|))
                av = expf(-(fmaxf(-zz, 0.f) + log1pf(expf(-fabsf(zz)))) * p.inv_tau);
            }
            sq[idx] = qv;
            sk[idx] = kv;
            sa[idx] = av;
        }
        for (int idx = tid; idx < nc * GLA_COLS; idx += GLA_THREADS) {
            int t = idx / GLA_COLS, c = idx - t * GLA_COLS;
            int cc = blockIdx.x * GLA_COLS + c;
            sv[idx] = cc < dv ? to_f32(vb[(size_t)(tok0 + c0 + t) * p.row_stride + h * dv + cc]) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nc; ++t) {
            const float vv = sv[t * GLA_COLS + cloc];
            const float* a = sa + t * DKP + part;
            const float* kk = sk + t * DKP + part;
            const float* qq = sq + t * DKP + part;
            float acc = 0.f;
#pragma unroll
            for (int m = 0; m < KPT; ++m) {
                S[m] = fmaf(a[GLA_KS * m], S[m], kk[GLA_KS * m] * vv);
                acc = fmaf(S[m], qq[GLA_KS * m], acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0 && col < dv) p.out[(size_t)(tok0 + c0 + t) * p.H * dv + h * dv + col] = acc;
        }
    }
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
        int i = part + GLA_KS * m;
        if (i < dk && col < dv) st[(size_t)i * dv + col] = S[m];
    }
}

template <typename T, int KPT>
static int launch_scan(const GlaParams& p, int B, cudaStream_t stream) {
    auto k = gla_scan_kernel<T, KPT>;
    size_t smem = (size_t)(3 * GLA_CHUNK * GLA_KS * KPT + GLA_CHUNK * GLA_COLS) * sizeof(float);
    dim3 grid((p.dv + GLA_COLS - 1) / GLA_COLS, p.H, B);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    llb_launch(k, grid, dim3(GLA_THREADS), smem, stream, p);
    return llb_status();
}

// Runs the recurrence over the new tokens of every sequence of the step and writes o [T, H * dv] (float32).
LLB_API int llb_gla_scan(GlaParams p, int dtype, int B, cudaStream_t stream) {
    if (B == 0) return 0;
    if (p.dk <= 0 || p.dv <= 0 || p.H <= 0 || p.dk > GLA_KS * 64) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, T, {
        if (p.dk <= GLA_KS * 8) return launch_scan<T, 8>(p, B, stream);
        if (p.dk <= GLA_KS * 16) return launch_scan<T, 16>(p, B, stream);
        if (p.dk <= GLA_KS * 32) return launch_scan<T, 32>(p, B, stream);
        return launch_scan<T, 64>(p, B, stream);
    });
    return 0;
}

// out[t, h * dv + d] = o[t, h, d] / sqrt(mean_d o[t, h, :]^2 + eps) * w[d] * silu(g[t, h * dv + d])
template <typename T, typename TW>
__global__ void __launch_bounds__(128) gla_out_kernel(const float* __restrict__ o, const T* __restrict__ g, int g_stride,
                                                      const TW* __restrict__ w, T* __restrict__ out, int rows, int H, int dv,
                                                      float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);       // (token, head)
    llb_grid_dependency_sync();
    if (r >= rows) return;
    const int t = r / H, h = r - t * H;
    const float* x = o + (size_t)r * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
        float gv = to_f32(g[(size_t)t * g_stride + h * dv + d]);
        out[(size_t)r * dv + d] = from_f32<T>(x[d] * inv * to_f32(w[d]) * (gv / (1.0f + expf(-gv))));
    }
}

LLB_API int llb_gla_out(const float* o, const void* g, int g_stride, const void* w, int w_dtype, void* out, int dtype,
                        int T, int H, int dv, float eps, cudaStream_t stream) {
    int rows = T * H;
    if (rows == 0) return 0;
    LLB_DISPATCH_DTYPE(dtype, TT, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            llb_launch(gla_out_kernel<TT, TW>, dim3((rows + 3) / 4), dim3(128), 0, stream, o, (const TT*)g, g_stride,
                       (const TW*)w, (TT*)out, rows, H, dv, eps);
        });
    });
    return llb_status();
}
