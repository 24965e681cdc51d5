// Kernels of the mixers, norms and activations beyond the rotary softmax attention of attention.cu:
//
//   dyntanh_kernel              y = tanh(alpha * (residual + x)) * w + b, the sum kept in the float32 stream
//   conv_norm_kvwrite_kernel    short causal convolution over time on q and k (carried per request in a state of the
//                               last taps-1 inputs), RMS norm over the whole q and the whole k projection, k and the
//                               un-normed k (the values) into the paged cache
//   conv_state_update_kernel    the state of that convolution after the step
//   window_attention_kernel     softmax attention over a sliding window plus the first tokens of the sequence, with a
//                               bias looked up by distance and one output gate per head; float32 arithmetic, any head size
//   decay_attention_kernel      linear attention with a fixed decay per head, S <- a S + k v^T, o = S^T q, the state in
//                               float32 per request; walks a request's tokens in order (decode and short portions)
//   decay_chunk_*_kernel        the same for long portions: chunks of a request in parallel, their sums scanned in order
//   rms_gate_kernel             RMS norm over a row, times sigmoid(gate), times a constant
//   gated_act_kernel            act(gate) * up with act = silu or tanh-gelu
//   head_gate_kernel            a head's output times the sigmoid of the head's gate, into packed rows
//   scaled_embedding_kernel     res = float(E[ids]) * c, the start of the float32 stream of a model that scales its embedding
//   postnorm_residual_kernel    res += c * rmsnorm(a) * w (a sublayer's output normed before it is added), and the next
//                               sublayer's input norm of the new stream in the same pass
//   latent_prep_kernel          latent attention: RMS norm of the query latent, RMS norm of the key/value latent and the
//                               rotation of the shared rotated key part, both into one row of the paged cache
//   rope_heads_kernel           the rotated part of every query head, angles from frequencies (no table, no position limit)
//   gated_decay_attention_kernel   linear attention whose decay is made from the input per token and key channel,
//                               S <- diag(alpha_t) S + k_t v_t^T, o = S^T q; token by token
//   gated_decay_chunk_*_kernel  the same for long portions, chunks of a request in parallel
//   group_rms_gate_kernel       RMS norm over each head of a row, times act(gate)
//
// Element type T (float or bfloat16) is the type of activations and caches; every sum, norm, score, weight of the
// softmax, decay and state is float32 in both.  Inputs that come out of a packed projection are addressed by a base
// pointer, a row stride and a column offset, outputs that go into a packed operand of the next product likewise.
#include "common.cuh"
#include <math.h>

#define MIX_MAX_TAPS 16

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}


// two neighbouring elements at once (V = 2) where pointers, strides and widths are even, else one (V = 1)
template <int V> __device__ __forceinline__ void ld_v(const float* p, float (&o)[2]) {
    if (V == 2) { const float2 t = *reinterpret_cast<const float2*>(p); o[0] = t.x; o[1] = t.y; } else { o[0] = p[0]; o[1] = 0.f; }
}
template <int V> __device__ __forceinline__ void ld_v(const __nv_bfloat16* p, float (&o)[2]) {
    if (V == 2) { const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p); o[0] = __low2float(t); o[1] = __high2float(t); }
    else { o[0] = __bfloat162float(p[0]); o[1] = 0.f; }
}
template <int V> __device__ __forceinline__ void st_v(float* p, const float (&o)[2]) {
    if (V == 2) *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]); else p[0] = o[0];
}
template <int V> __device__ __forceinline__ void st_v(__nv_bfloat16* p, const float (&o)[2]) {
    if (V == 2) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o[0], o[1]); else p[0] = __float2bfloat16_rn(o[0]);
}
// V neighbouring elements at once, V = 1, 2 or 8 (8: 16 bytes of bfloat16, two 16-byte pieces of float32)
template <int V> __device__ __forceinline__ void ld_w(const float* p, float (&o)[V]) {
    if constexpr (V == 8) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    } else if constexpr (V == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p); o[0] = t.x; o[1] = t.y;
    } else {
        o[0] = p[0];
    }
}
template <int V> __device__ __forceinline__ void ld_w(const __nv_bfloat16* p, float (&o)[V]) {
    if constexpr (V == 8) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            o[2 * i] = __low2float(h); o[2 * i + 1] = __high2float(h);
        }
    } else if constexpr (V == 2) {
        const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p); o[0] = __low2float(t); o[1] = __high2float(t);
    } else {
        o[0] = __bfloat162float(p[0]);
    }
}
template <int V> __device__ __forceinline__ void st_w(float* p, const float (&o)[V]) {
    if constexpr (V == 8) {
        *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
    } else if constexpr (V == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]);
    } else {
        p[0] = o[0];
    }
}
template <int V> __device__ __forceinline__ void st_w(__nv_bfloat16* p, const float (&o)[V]) {
    if constexpr (V == 8) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if constexpr (V == 2) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o[0], o[1]);
    } else {
        p[0] = __float2bfloat16_rn(o[0]);
    }
}
static inline bool multiple_of(long long m, long long a, long long b = 0, long long c = 0, long long d = 0, long long e = 0, long long f = 0) {
    return a % m == 0 && b % m == 0 && c % m == 0 && d % m == 0 && e % m == 0 && f % m == 0;
}
static inline bool even_all(long long a, long long b = 0, long long c = 0, long long d = 0, long long e = 0, long long f = 0) {
    return ((a | b | c | d | e | f) & 1) == 0;
}
static inline bool aligned_to(const void* p, size_t n) { return p == nullptr || ((uintptr_t)p % n) == 0; }

// ---------------------------------------------------------------------------------------
// Dynamic Tanh norm
// ---------------------------------------------------------------------------------------
template <typename T, typename X, int V>
__global__ void dyntanh_kernel(const X* __restrict__ x, const float* __restrict__ res_in, float* __restrict__ res_out,
                               const int* __restrict__ row_idx, const float* __restrict__ w, const float* __restrict__ b,
                               float alpha, T* __restrict__ y, int H) {
    const int i = blockIdx.x;
    const size_t r = row_idx ? (size_t)row_idx[i] : (size_t)i;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * V; c < H; c += gridDim.y * blockDim.x * V) {
        float v[2] = {0.f, 0.f}, xv[2] = {0.f, 0.f}, wv[2], bv[2], o[2];
        if (res_in) ld_v<V>(res_in + r * H + c, v);
        if (x) { ld_v<V>(x + r * H + c, xv); v[0] += xv[0]; v[1] += xv[1]; }
        if (res_out) st_v<V>(res_out + r * H + c, v);
        ld_v<V>(w + c, wv);
        ld_v<V>(b + c, bv);
        o[0] = tanhf(alpha * v[0]) * wv[0] + bv[0];
        o[1] = V == 2 ? tanhf(alpha * v[1]) * wv[1] + bv[1] : 0.f;
        st_v<V>(y + (size_t)i * H + c, o);
    }
}

template <typename T, typename X>
static void dyntanh_launch(const void* x, const float* res_in, float* res_out, const int* row_idx, const float* w, const float* b,
                           float alpha, void* y, int rows, int H, cudaStream_t stream) {
    const bool v2 = even_all(H) && aligned_to(x, 2 * sizeof(X)) && aligned_to(res_in, 8) && aligned_to(res_out, 8) && aligned_to(w, 8) &&
                    aligned_to(b, 8) && aligned_to(y, 2 * sizeof(T));
    const int per = v2 ? 2 : 1;
    const dim3 grid(rows, max(1, min((H + 128 * per - 1) / (128 * per), 32)));
    if (v2) dyntanh_kernel<T, X, 2><<<grid, 128, 0, stream>>>((const X*)x, res_in, res_out, row_idx, w, b, alpha, (T*)y, H);
    else dyntanh_kernel<T, X, 1><<<grid, 128, 0, stream>>>((const X*)x, res_in, res_out, row_idx, w, b, alpha, (T*)y, H);
}

MSGL_API int msgl_dyntanh(const void* x, int x_is_f32, const float* res_in, float* res_out, const int* row_idx,
                          const float* w, const float* b, float alpha, void* y, int rows, int H, int dtype,
                          cudaStream_t stream) {
    if (rows <= 0) return MSGL_OK;
    if (H <= 0) return MSGL_ERR_SIZE;
    if (dtype == MSGL_F32) dyntanh_launch<float, float>(x, res_in, res_out, row_idx, w, b, alpha, y, rows, H, stream);
    else if (dtype == MSGL_BF16 && x_is_f32) dyntanh_launch<__nv_bfloat16, float>(x, res_in, res_out, row_idx, w, b, alpha, y, rows, H, stream);
    else if (dtype == MSGL_BF16) dyntanh_launch<__nv_bfloat16, __nv_bfloat16>(x, res_in, res_out, row_idx, w, b, alpha, y, rows, H, stream);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Short causal convolution on q and k + whole-projection RMS norm + cache write
//
//   proj row: q at column q_off (Cq = heads * d channels), k at column k_off (Ck = kv heads * d)
//   y[t, c] = sum_j w[j, c] * u[t - taps + 1 + j, c] (the taps' weights come transposed, [taps][channels]); inputs before this step's first token come from the
//   request's state [slot][taps - 1][Cq + Ck] (oldest first; zero when the request was opened)
//   q_out = rms(y_q) * wq_norm;  K cache <- rms(y_k) * wk_norm;  V cache <- y_k (before the norm)
// One block per token.
// ---------------------------------------------------------------------------------------
struct ConvNormParams {
    const void* proj; long long stride; int q_off, k_off;
    int Cq, Ck, d, n_kv, taps;
    const float* wq_conv; const float* wk_conv;      // [taps, C]: a tap's weights of neighbouring channels side by side
    const float* wq_norm; const float* wk_norm;      // [C]
    float eps;
    void* state;                                     // [slots][taps - 1][Cq + Ck]
    const int* token_req; const int* q_start; const int* slots; const int* out_loc;
    void* q_out;                                     // [T, Cq]
    void* k_cache; void* v_cache; int page_size;
    int T;
    int one_token;                                   // every request brings one token: its block brings the state up to date itself
};

template <typename T, int V, int KMAX /* most taps: 4 or MIX_MAX_TAPS */>
__global__ void __launch_bounds__(KMAX <= 4 ? 1024 : 256) conv_norm_kvwrite_kernel(const ConvNormParams p) {
    extern __shared__ __align__(16) float ybuf[];    // [Cq + Ck]
    __shared__ float red[64];
    const int t = blockIdx.x;
    // one token a request: token t is request t's only one, no lookups
    const int r = p.one_token ? t : p.token_req[t];
    const int t0 = p.one_token ? t : p.q_start[r];
    const int i = t - t0;                            // index of the token within the request's tokens of this step
    const int slot = p.slots[r];
    const int C = p.Cq + p.Ck, K = p.taps;
    const T* proj = reinterpret_cast<const T*>(p.proj);
    const T* st = reinterpret_cast<const T*>(p.state) + (size_t)slot * (K - 1) * C;
    float ssq_q = 0.f, ssq_k = 0.f;
    for (int c = threadIdx.x * V; c < C; c += blockDim.x * V) {
        const bool is_q = c < p.Cq;
        const int cc = is_q ? c : c - p.Cq;
        const float* w = (is_q ? p.wq_conv : p.wk_conv) + cc;
        const int Cw = is_q ? p.Cq : p.Ck;
        const int col = is_q ? p.q_off + cc : p.k_off + cc;
        // every input of the taps first, then the sums: the loads are in flight together
        float u[KMAX][V];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            if (j < K) {
                const int idx = i - (K - 1) + j;     // relative to the step's first token of this request
                if (idx >= 0) ld_w<V>(proj + (size_t)(t0 + idx) * p.stride + col, u[j]);
                else ld_w<V>(st + (size_t)(K - 1 + idx) * C + c, u[j]);
            }
        }
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            if (j < K) {
                float wv[V];
                ld_w<V>(w + (size_t)j * Cw, wv);
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = fmaf(wv[v], u[j][v], acc[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            acc[v] = to_f32<T>(from_f32<T>(acc[v]));          // as it leaves the convolution, in the activation type
            if (is_q) ssq_q += acc[v] * acc[v]; else ssq_k += acc[v] * acc[v];
        }
        st_w<V>(ybuf + c, acc);
    }
    // both sums over the block at once
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        ssq_q = warp_sum(ssq_q);
        ssq_k = warp_sum(ssq_k);
        if (lane == 0) { red[warp] = ssq_q; red[32 + warp] = ssq_k; }
        __syncthreads();
        const int nwarps = (blockDim.x + 31) >> 5;
        ssq_q = warp_sum(lane < nwarps ? red[lane] : 0.f);
        ssq_k = warp_sum(lane < nwarps ? red[32 + lane] : 0.f);
    }
    const float rq = 1.f / sqrtf(ssq_q / (float)p.Cq + p.eps), rk = 1.f / sqrtf(ssq_k / (float)p.Ck + p.eps);
    T* qo = reinterpret_cast<T*>(p.q_out) + (size_t)t * p.Cq;
    const int loc = p.out_loc ? p.out_loc[t] : 0;
    const int page = loc / p.page_size, ps = loc - page * p.page_size;
    T* kc = reinterpret_cast<T*>(p.k_cache);
    T* vc = reinterpret_cast<T*>(p.v_cache);
    for (int c = threadIdx.x * V; c < C; c += blockDim.x * V) {      // a thread reads back what it wrote itself
        float y[V], o[V], wn[V];
        ld_w<V>(ybuf + c, y);
        if (c < p.Cq) {
            ld_w<V>(p.wq_norm + c, wn);
#pragma unroll
            for (int v = 0; v < V; ++v) o[v] = y[v] * rq * wn[v];
            st_w<V>(qo + c, o);
        } else if (kc) {
            const int cc = c - p.Cq;
            const int g = cc / p.d, e = cc - g * p.d;
            const size_t a = (((size_t)page * p.n_kv + g) * p.page_size + ps) * p.d + e;
            ld_w<V>(p.wk_norm + cc, wn);
#pragma unroll
            for (int v = 0; v < V; ++v) o[v] = y[v] * rk * wn[v];
            st_w<V>(kc + a, o);
            st_w<V>(vc + a, y);
        }
    }
    if (p.one_token && K > 1) {
        // the request's only token of the step: its state moves up by one row.  A thread moves the channels it summed itself,
        // row by row from the oldest, so every row is read before it is written; all reads of the sums lie behind the barrier.
        T* stw = reinterpret_cast<T*>(p.state) + (size_t)slot * (K - 1) * C;
        for (int c = threadIdx.x * V; c < C; c += blockDim.x * V) {
            const int col = c < p.Cq ? p.q_off + c : p.k_off + (c - p.Cq);
            float v[V];
            for (int k = 0; k + 1 < K - 1; ++k) {
                ld_w<V>(stw + (size_t)(k + 1) * C + c, v);
                st_w<V>(stw + (size_t)k * C + c, v);
            }
            ld_w<V>(proj + (size_t)t * p.stride + col, v);
            st_w<V>(stw + (size_t)(K - 2) * C + c, v);
        }
    }
}

template <typename T>
__global__ void conv_state_update_kernel(const void* proj_, long long stride, int q_off, int k_off, int Cq, int Ck, int taps,
                                         void* state_, const int* __restrict__ q_start, const int* __restrict__ slots) {
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int C = Cq + Ck, K = taps;
    if (c >= C) return;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    const int slot = slots[r];
    const T* proj = reinterpret_cast<const T*>(proj_);
    T* st = reinterpret_cast<T*>(state_) + (size_t)slot * (K - 1) * C;
    const int col = c < Cq ? q_off + c : k_off + (c - Cq);
    T keep[MIX_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MIX_MAX_TAPS; ++k) {
        if (k < K - 1) {
            const int idx = n - (K - 1) + k;         // index among this step's tokens of the request; negative: older
            keep[k] = idx >= 0 ? proj[(size_t)(t0 + idx) * stride + col] : st[(size_t)(K - 1 + idx) * C + c];
        }
    }
#pragma unroll
    for (int k = 0; k < MIX_MAX_TAPS; ++k)
        if (k < K - 1) st[(size_t)k * C + c] = keep[k];
}

MSGL_API int msgl_conv_norm_kvwrite(const void* proj, long long stride, int q_off, int k_off, int Cq, int Ck, int d, int n_kv,
                                    int taps, const float* wq_conv, const float* wk_conv, const float* wq_norm,
                                    const float* wk_norm, float eps, void* state, const int* token_req, const int* q_start,
                                    const int* slots, const int* out_loc, void* q_out, void* k_cache, void* v_cache,
                                    int page_size, int T, int B, int one_token, int dtype, cudaStream_t stream) {
    if (T <= 0) return MSGL_OK;
    if (taps < 1 || taps > MIX_MAX_TAPS || Cq <= 0 || Ck <= 0 || d <= 0 || Ck != n_kv * d) return MSGL_ERR_SIZE;
    ConvNormParams p;
    p.proj = proj; p.stride = stride; p.q_off = q_off; p.k_off = k_off; p.Cq = Cq; p.Ck = Ck; p.d = d; p.n_kv = n_kv; p.taps = taps;
    p.wq_conv = wq_conv; p.wk_conv = wk_conv; p.wq_norm = wq_norm; p.wk_norm = wk_norm; p.eps = eps; p.state = state;
    p.token_req = token_req; p.q_start = q_start; p.slots = slots; p.out_loc = out_loc; p.q_out = q_out;
    p.k_cache = k_cache; p.v_cache = v_cache; p.page_size = page_size; p.T = T;
    p.one_token = (one_token && T == B) ? 1 : 0;
    const size_t smem = (size_t)(Cq + Ck) * sizeof(float);
    if (smem > 200 * 1024) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const size_t item = dtype == MSGL_F32 ? 4 : 2;
    // pairs of channels where nothing is odd: widths, head size, offsets, strides, pointers
    const bool v2 = even_all(Cq, Ck, d, q_off, k_off, stride) && aligned_to(proj, 2 * item) && aligned_to(state, 2 * item) &&
                    aligned_to(q_out, 2 * item) && aligned_to(k_cache, 2 * item) && aligned_to(v_cache, 2 * item) &&
                    aligned_to(wq_norm, 8) && aligned_to(wk_norm, 8) && aligned_to(wq_conv, 8) && aligned_to(wk_conv, 8);
    // eight channels at once where everything is a multiple of eight and 16-byte aligned
    const bool v8 = v2 && multiple_of(8, Cq, Ck, d, q_off, k_off, stride) && aligned_to(proj, 16) && aligned_to(state, 16) &&
                    aligned_to(q_out, 16) && aligned_to(k_cache, 16) && aligned_to(v_cache, 16) && aligned_to(wq_norm, 32) &&
                    aligned_to(wk_norm, 32) && aligned_to(wq_conv, 32) && aligned_to(wk_conv, 32);
    const int per = v8 ? 8 : (v2 ? 2 : 1);
    const int C = Cq + Ck;
    const bool few = taps <= 4;
    // many tokens: small blocks, several a multiprocessor, so that one block's loads overlap another's sums and stores; few
    // tokens: one large block a token
    const int threads = (!few || T >= 256) ? (C / per >= 512 ? 256 : 128) : (C / per >= 2048 ? 1024 : (C / per >= 512 ? 512 : 256));
#define CONV_LAUNCH(T, V, KM)                                                                                         \
    do {                                                                                                              \
        static MsglOncePerDevice once;                                                                                \
        if (smem > 48 * 1024 && once.due()) {                                                                         \
            cudaFuncSetAttribute(conv_norm_kvwrite_kernel<T, V, KM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            once.mark();                                                                                              \
        }                                                                                                             \
        conv_norm_kvwrite_kernel<T, V, KM><<<T_, threads, smem, stream>>>(p);                                         \
    } while (0)
#define CONV_LAUNCH_K(T, V) do { if (few) CONV_LAUNCH(T, V, 4); else CONV_LAUNCH(T, V, MIX_MAX_TAPS); } while (0)
    const int T_ = T;
    if (dtype == MSGL_F32) { if (v8) CONV_LAUNCH_K(float, 8); else if (v2) CONV_LAUNCH_K(float, 2); else CONV_LAUNCH_K(float, 1); }
    else { if (v8) CONV_LAUNCH_K(__nv_bfloat16, 8); else if (v2) CONV_LAUNCH_K(__nv_bfloat16, 2); else CONV_LAUNCH_K(__nv_bfloat16, 1); }
#undef CONV_LAUNCH_K
#undef CONV_LAUNCH
    if (taps > 1 && !p.one_token) {
        const dim3 grid(B, (C + 255) / 256);
        if (dtype == MSGL_F32)
            conv_state_update_kernel<float><<<grid, 256, 0, stream>>>(proj, stride, q_off, k_off, Cq, Ck, taps, state, q_start, slots);
        else
            conv_state_update_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(proj, stride, q_off, k_off, Cq, Ck, taps, state, q_start, slots);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Softmax attention over a window and the first tokens, with a bias by distance and an output gate
//
//   query at position i sees key j if j <= i and (i - j < window or j < keep_first)
//   score = q . k * scale + bias[head][min(i - j, L - 1)]
//   out[t, head, :] = softmax(score) V * sigmoid(gate[t, head]) * out_scale
//
// A block takes QT consecutive tokens of one request and GH query heads of one kv head: QT * GH <= 8 rows, one warp
// each.  Keys go through shared memory in chunks of 32 anchored at multiples of 32, first the chunks that hold kept first
// tokens before the window, then the window's, in rising order: the order of the sums at a position does not depend on
// how the tokens were cut into steps.  In the score phase lane l of a row's warp takes key l of the chunk; in the value
// phase lane l takes the output elements l, l + 32, ...
// ---------------------------------------------------------------------------------------
#define WA_ROWS 8
#define WA_KC 32
#define WA_MAX_DPL 16       // head sizes up to 512

struct WindowAttnParams {
    const void* q;            // [T, n_q, d]
    const void* k_cache; const void* v_cache;
    const int* q_start; const int* kv_len; const int* block_table; int bt_stride;
    int uniform;                                  // every request brings one token: block x takes request x
    const float* bias; int bias_len;              // [n_q][bias_len] or null
    const void* gate; long long gate_stride; int gate_off;        // [T rows][.. n_q at gate_off] or null
    void* out; long long out_stride; int out_off;                 // [T rows][.. n_q * d at out_off]
    int B, n_q, n_kv, d, page_size, window, keep_first, QT, GH;
    float scale, out_scale;
};

template <typename T, int DPL /* output elements per lane: head sizes up to 32 * DPL */>
__global__ void __launch_bounds__(WA_ROWS * 32) window_attention_kernel(const WindowAttnParams p) {
    extern __shared__ float smem[];
    const int d = p.d;
    float* qs = smem;                                // [WA_ROWS][d]
    float* ks = qs + WA_ROWS * d;                    // [WA_KC][d + 1]
    float* vs = ks + WA_KC * (d + 1);                // [WA_KC][d]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // block x is the x-th query tile of the step: tiles of QT tokens, request by request
    __shared__ int tile_sh[2];
    int req, t0;
    if (p.uniform) {
        req = blockIdx.x; t0 = 0;
    } else {
        if (tid == 0) {
            int left = blockIdx.x, found = -1, at = 0;
            for (int r = 0; r < p.B; ++r) {
                const int nt = (p.q_start[r + 1] - p.q_start[r] + p.QT - 1) / p.QT;
                if (left < nt) { found = r; at = left * p.QT; break; }
                left -= nt;
            }
            tile_sh[0] = found; tile_sh[1] = at;
        }
        __syncthreads();
        req = tile_sh[0]; t0 = tile_sh[1];
    }
    if (req < 0 || req >= p.B) return;
    const int G = p.n_q / p.n_kv;
    const int n_chunks = (G + p.GH - 1) / p.GH;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    const int q_base = p.q_start[req], q_len = p.q_start[req + 1] - q_base, kv_len = p.kv_len[req];
    const int n_tok = min(p.QT, q_len - t0);
    if (n_tok <= 0) return;
    const int p_min = kv_len - q_len + t0, p_max = p_min + n_tok - 1;
    const int window = p.window > 0 ? p.window : (1 << 30);
    const int win_lo = max(0, p_min - window + 1);
    const int sink_hi = min(p.keep_first, win_lo);                 // kept first tokens that lie before the tile's window
    const int c_first = win_lo / WA_KC, c_last = p_max / WA_KC;
    const int n_sink = min((sink_hi + WA_KC - 1) / WA_KC, c_first);
    const int n_c = n_sink + (c_last - c_first + 1);

    // this warp's row
    const int tl = warp / p.GH, hl = warp - tl * p.GH;
    const int hg = chunk * p.GH + hl;
    const bool row_ok = tl < n_tok && hg < G && tl < p.QT;
    const int head = kvh * G + (row_ok ? hg : 0);
    const int tok = q_base + t0 + (row_ok ? tl : 0);
    const int pos = p_min + tl;
    const T* qg = reinterpret_cast<const T*>(p.q);
    for (int e = lane; e < d; e += 32) qs[warp * d + e] = row_ok ? to_f32<T>(qg[((size_t)tok * p.n_q + head) * d + e]) : 0.f;
    const float* bias = p.bias ? p.bias + (size_t)head * p.bias_len : nullptr;

    const T* kc = reinterpret_cast<const T*>(p.k_cache);
    const T* vc = reinterpret_cast<const T*>(p.v_cache);
    const int* bt = p.block_table + (size_t)req * p.bt_stride;

    float o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int ci = 0; ci < n_c; ++ci) {
        const int c = ci < n_sink ? ci : c_first + (ci - n_sink);
        const int key0 = c * WA_KC;
        __syncthreads();
        // ---- the chunk's keys and values into shared memory (rows past the last key: zeros)
        for (int idx = tid; idx < WA_KC * d; idx += WA_ROWS * 32) {
            const int kr = idx / d, e = idx - kr * d;
            const int key = key0 + kr;
            float kv = 0.f, vv = 0.f;
            if (key <= p_max) {
                const int page = bt[key / p.page_size];
                const size_t a = (((size_t)page * p.n_kv + kvh) * p.page_size + (key % p.page_size)) * d + e;
                kv = to_f32<T>(kc[a]);
                vv = to_f32<T>(vc[a]);
            }
            ks[kr * (d + 1) + e] = kv;
            vs[kr * d + e] = vv;
        }
        __syncthreads();
        // ---- score of key `lane`
        const int key = key0 + lane;
        const bool vis = row_ok && key <= pos && (pos - key < window || key < p.keep_first);
        float s = -INFINITY;
        if (vis) {
            float acc = 0.f;
            const float* qr = qs + warp * d;
            const float* kr = ks + lane * (d + 1);
            for (int e = 0; e < d; ++e) acc = fmaf(qr[e], kr[e], acc);
            s = acc * p.scale;
            if (bias) s += bias[min(pos - key, p.bias_len - 1)];
        }
        const float cmax = warp_max(s);
        if (cmax == -INFINITY) continue;             // no key of this chunk is visible from this row (warp-uniform)
        const float m_new = fmaxf(m, cmax);
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = vis ? expf(s - m_new) : 0.f;
        l = l * alpha + pr;
        m = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= alpha;
        // ---- values
        for (int j = 0; j < WA_KC; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            if (pj == 0.f) continue;                 // warp-uniform
            const float* vr = vs + j * d;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < d) o[i] = fmaf(pj, vr[e], o[i]);
            }
        }
    }
    l = warp_sum(l);
    if (!row_ok) return;
    float f = (l > 0.f ? 1.f / l : 0.f) * p.out_scale;
    if (p.gate) {
        const T* gg = reinterpret_cast<const T*>(p.gate);
        f *= sigmoidf_(to_f32<T>(gg[(size_t)tok * p.gate_stride + p.gate_off + head]));
    }
    T* og = reinterpret_cast<T*>(p.out) + (size_t)tok * p.out_stride + p.out_off + (size_t)head * d;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < d) og[e] = from_f32<T>(o[i] * f);
    }
}

MSGL_API int msgl_window_attention(const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len,
                                   const int* block_table, int bt_stride, int uniform, int n_tiles,
                                   const float* bias, int bias_len, const void* gate, long long gate_stride, int gate_off,
                                   void* out, long long out_stride, int out_off, int B, int n_q, int n_kv, int d, int page_size,
                                   int window, int keep_first, int QT, int GH, float scale, float out_scale, int dtype,
                                   cudaStream_t stream) {
    if (n_tiles <= 0) return MSGL_OK;
    if (d <= 0 || d > 32 * WA_MAX_DPL || n_kv <= 0 || n_q % n_kv || QT < 1 || GH < 1 || QT * GH > WA_ROWS || page_size < 1)
        return MSGL_ERR_SIZE;
    WindowAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.bt_stride = bt_stride; p.uniform = uniform; p.bias = bias; p.bias_len = bias_len; p.gate = gate;
    p.gate_stride = gate_stride; p.gate_off = gate_off; p.out = out; p.out_stride = out_stride; p.out_off = out_off; p.B = B;
    p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.page_size = page_size; p.window = window; p.keep_first = keep_first; p.QT = QT;
    p.GH = GH; p.scale = scale; p.out_scale = out_scale;
    const int G = n_q / n_kv;
    const dim3 grid(n_tiles, n_kv * ((G + GH - 1) / GH));
    const size_t smem = ((size_t)WA_ROWS * d + (size_t)WA_KC * (d + 1) + (size_t)WA_KC * d) * sizeof(float);
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int dpl = (d + 31) / 32;
#define WA_LAUNCH(N)                                                                                                        \
    do {                                                                                                                    \
        static MsglOncePerDevice once;                                                                                      \
        if (smem > 48 * 1024 && once.due()) {                                                                               \
            cudaFuncSetAttribute(window_attention_kernel<float, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            cudaFuncSetAttribute(window_attention_kernel<__nv_bfloat16, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            once.mark();                                                                                                    \
        }                                                                                                                   \
        if (dtype == MSGL_F32) window_attention_kernel<float, N><<<grid, WA_ROWS * 32, smem, stream>>>(p);                  \
        else window_attention_kernel<__nv_bfloat16, N><<<grid, WA_ROWS * 32, smem, stream>>>(p);                            \
    } while (0)
    if (dpl <= 1) WA_LAUNCH(1);
    else if (dpl <= 2) WA_LAUNCH(2);
    else if (dpl <= 3) WA_LAUNCH(3);
    else if (dpl <= 4) WA_LAUNCH(4);
    else if (dpl <= 8) WA_LAUNCH(8);
    else WA_LAUNCH(16);
#undef WA_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Linear attention with a fixed decay per head
//
//   q = silu(proj q), k = silu(proj k) [heads][dk], v = silu(proj v) [heads][dv]
//   S_t = decay_h * S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  S per request [slot][heads][dk][dv] float32
//
// A block owns 32 columns of one (request, head) state and walks the request's tokens of the step in order; the
// column's dk rows are dealt out to 8 neighbouring lanes, which add their parts of o with shuffles.
// ---------------------------------------------------------------------------------------
#define DA_COLS 32
#define DA_PARTS 8
#define DA_MAX_ROWS 64      // most rows of a column per lane: key sizes up to 512

template <typename T, int NR /* rows of a column per lane: key sizes up to DA_PARTS * NR */>
__global__ void __launch_bounds__(DA_COLS * DA_PARTS)
decay_attention_kernel(const void* proj_, long long stride, int q_off, int k_off, int v_off, int heads, int dk, int dv,
                       const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ q_start,
                       const int* __restrict__ slots, float* __restrict__ out /* [T, heads * dv] */) {
    extern __shared__ float qk[];                    // [2][2][dk]: double-buffered q and k of the current token
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DA_COLS;
    const int tid = threadIdx.x;
    const int part = tid & (DA_PARTS - 1), col = col0 + (tid >> 3);
    const bool col_ok = col < dv;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    const int slot = slots[r];
    const float a = decay[h];
    const T* proj = reinterpret_cast<const T*>(proj_);
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    const int rows = (dk + DA_PARTS - 1) / DA_PARTS;             // rows i = part + DA_PARTS * j
    float s[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + DA_PARTS * j;
        s[j] = (j < rows && i < dk && col_ok) ? S[(size_t)i * dv + col] : 0.f;
    }
    for (int tt = 0; tt < n; ++tt) {
        const size_t row = (size_t)(t0 + tt) * stride;
        float* qb = qk + (tt & 1) * 2 * dk;
        float* kb = qb + dk;
        for (int i = tid; i < 2 * dk; i += DA_COLS * DA_PARTS) {
            const int c = i < dk ? q_off + h * dk + i : k_off + h * dk + (i - dk);
            qb[i] = siluf_(to_f32<T>(proj[row + c]));
        }
        const float v = col_ok ? siluf_(to_f32<T>(proj[row + v_off + h * dv + col])) : 0.f;
        __syncthreads();
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            if (j < rows) {
                const int i = part + DA_PARTS * j;
                if (i < dk) {
                    s[j] = fmaf(a, s[j], kb[i] * v);
                    acc = fmaf(s[j], qb[i], acc);
                }
            }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (part == 0 && col_ok) out[(size_t)(t0 + tt) * heads * dv + h * dv + col] = acc;
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + DA_PARTS * j;
        if (j < rows && i < dk && col_ok) S[(size_t)i * dv + col] = s[j];
    }
}

MSGL_API int msgl_decay_attention(const void* proj, long long stride, int q_off, int k_off, int v_off, int heads, int dk, int dv,
                                  const float* decay, float* state, const int* q_start, const int* slots, float* out, int B,
                                  int dtype, cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0 || dk > DA_PARTS * DA_MAX_ROWS) return MSGL_ERR_SIZE;
    const dim3 grid(B, heads, (dv + DA_COLS - 1) / DA_COLS);
    const size_t smem = (size_t)4 * dk * sizeof(float);
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int nr = (dk + DA_PARTS - 1) / DA_PARTS;
#define DA_LAUNCH(N)                                                                                                                 \
    do {                                                                                                                             \
        if (dtype == MSGL_F32)                                                                                                       \
            decay_attention_kernel<float, N><<<grid, DA_COLS * DA_PARTS, smem, stream>>>(proj, stride, q_off, k_off, v_off, heads, dk, \
                                                                                         dv, decay, state, q_start, slots, out);   \
        else                                                                                                                         \
            decay_attention_kernel<__nv_bfloat16, N><<<grid, DA_COLS * DA_PARTS, smem, stream>>>(proj, stride, q_off, k_off, v_off,    \
                                                                                                 heads, dk, dv, decay, state,      \
                                                                                                 q_start, slots, out);             \
    } while (0)
    if (nr <= 4) DA_LAUNCH(4);
    else if (nr <= 8) DA_LAUNCH(8);
    else if (nr <= 16) DA_LAUNCH(16);
    else if (nr <= 32) DA_LAUNCH(32);
    else DA_LAUNCH(64);
#undef DA_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The same linear attention for long portions: a request's tokens of the step in chunks of 64, the chunks in parallel.
// With L tokens in a chunk (local index i), a the head's decay and S the state before the chunk:
//
//   1. decay_chunk_kv_kernel    U = sum_i a^(L-1-i) k_i v_i^T                      every chunk by itself
//   2. decay_chunk_scan_kernel  per request, chunk after chunk: U <- S (the state before the chunk), S <- a^L S + U;
//                               the request's state row gets the last S
//   3. decay_chunk_out_kernel   o_i = a^(i+1) S^T q_i + sum_{j<=i} a^(i-j) (q_i . k_j) v_j
//
// All products are float32 FMA on 64 x 64 tiles through shared memory, 4 x 4 results a thread.
// ---------------------------------------------------------------------------------------
#define DC_C 64
#define DC_LD 65

struct DecayChunkParams {
    const void* proj; long long stride; int q_off, k_off, v_off;
    int heads, dk, dv, B;
    const float* decay; float* state; const int* q_start; const int* slots;
    float* U;       // [chunks][heads][dk][dv]
    float* out;     // [T][heads * dv]
};

__device__ __forceinline__ float dc_pow(float log2a, int n) { return n == 0 ? 1.f : exp2f((float)n * log2a); }

// chunk index -> (request, first token of the chunk among the step's tokens, tokens in the chunk); false: no such chunk
__device__ __forceinline__ bool dc_find_chunk(const DecayChunkParams& p, int chunk, int* sh, int& req, int& t0, int& L) {
    if (threadIdx.x == 0) {
        int left = chunk, found = -1, c0 = 0;
        for (int r = 0; r < p.B; ++r) {
            const int nc = (p.q_start[r + 1] - p.q_start[r] + DC_C - 1) / DC_C;
            if (left < nc) { found = r; c0 = left * DC_C; break; }
            left -= nc;
        }
        sh[0] = found; sh[1] = c0;
    }
    __syncthreads();
    req = sh[0];
    if (req < 0) return false;
    const int base = p.q_start[req], n = p.q_start[req + 1] - base;
    t0 = base + sh[1];
    L = min(DC_C, n - sh[1]);
    return true;
}

template <typename T>
__global__ void __launch_bounds__(256) decay_chunk_kv_kernel(const DecayChunkParams p) {
    __shared__ __align__(16) float Ks[DC_C][64];
    __shared__ __align__(16) float Vs[DC_C][64];
    __shared__ int sh[2];
    const int chunk = blockIdx.x, h = blockIdx.y;
    const int n_ct = (p.dv + 63) / 64;
    const int row0 = (blockIdx.z / n_ct) * 64, col0 = (blockIdx.z % n_ct) * 64;
    int req, t0, L;
    if (!dc_find_chunk(p, chunk, sh, req, t0, L)) return;
    const float la = log2f(p.decay[h]);
    const T* proj = reinterpret_cast<const T*>(p.proj);
    const int tid = threadIdx.x;
    for (int idx = tid; idx < DC_C * 64; idx += 256) {
        const int i = idx >> 6, m = idx & 63;
        float kv = 0.f, vv = 0.f;
        if (i < L) {
            const size_t row = (size_t)(t0 + i) * p.stride;
            if (row0 + m < p.dk) kv = siluf_(to_f32<T>(proj[row + p.k_off + h * p.dk + row0 + m])) * dc_pow(la, L - 1 - i);
            if (col0 + m < p.dv) vv = siluf_(to_f32<T>(proj[row + p.v_off + h * p.dv + col0 + m]));
        }
        Ks[i][m] = kv;
        Vs[i][m] = vv;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4] = {};
    for (int i = 0; i < L; ++i) {
        const float4 kr = *reinterpret_cast<const float4*>(&Ks[i][ty * 4]);
        const float4 vr = *reinterpret_cast<const float4*>(&Vs[i][tx * 4]);
        const float ka[4] = {kr.x, kr.y, kr.z, kr.w}, va[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ka[a], va[b], acc[a][b]);
    }
    float* U = p.U + ((size_t)chunk * p.heads + h) * p.dk * p.dv;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int row = row0 + ty * 4 + a;
        if (row >= p.dk) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int col = col0 + tx * 4 + b;
            if (col < p.dv) U[(size_t)row * p.dv + col] = acc[a][b];
        }
    }
}

__global__ void decay_chunk_scan_kernel(const DecayChunkParams p) {
    const int r = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int E = p.dk * p.dv;
    if (e >= E) return;
    const int n = p.q_start[r + 1] - p.q_start[r];
    if (n <= 0) return;
    int chunk0 = 0;
    for (int r2 = 0; r2 < r; ++r2) chunk0 += (p.q_start[r2 + 1] - p.q_start[r2] + DC_C - 1) / DC_C;
    const float la = log2f(p.decay[h]);
    float* st = p.state + ((size_t)p.slots[r] * p.heads + h) * E + e;
    float S = *st;
    const int nc = (n + DC_C - 1) / DC_C;
    for (int c = 0; c < nc; ++c) {
        const int L = min(DC_C, n - c * DC_C);
        float* u = p.U + ((size_t)(chunk0 + c) * p.heads + h) * E + e;
        const float uv = *u;
        *u = S;
        S = fmaf(dc_pow(la, L), S, uv);
    }
    *st = S;
}

template <typename T>
__global__ void __launch_bounds__(256) decay_chunk_out_kernel(const DecayChunkParams p) {
    __shared__ __align__(16) float As[DC_C][DC_LD];       // q slab; then v
    __shared__ __align__(16) float Bs[DC_C][DC_LD];       // k slab; then the chunk's weights P; then a slab of S
    __shared__ int sh[2];
    const int chunk = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * 64;
    int req, t0, L;
    if (!dc_find_chunk(p, chunk, sh, req, t0, L)) return;
    const float la = log2f(p.decay[h]);
    const T* proj = reinterpret_cast<const T*>(p.proj);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;

    // ---- P[i][j] = a^(i-j) q_i . k_j for j <= i
    float pacc[4][4] = {};
    for (int m0 = 0; m0 < p.dk; m0 += 64) {
        __syncthreads();
        for (int idx = tid; idx < DC_C * 64; idx += 256) {
            const int i = idx >> 6, m = idx & 63;
            float qv = 0.f, kv = 0.f;
            if (i < L && m0 + m < p.dk) {
                const size_t row = (size_t)(t0 + i) * p.stride;
                qv = siluf_(to_f32<T>(proj[row + p.q_off + h * p.dk + m0 + m]));
                kv = siluf_(to_f32<T>(proj[row + p.k_off + h * p.dk + m0 + m]));
            }
            As[i][m] = qv;
            Bs[i][m] = kv;
        }
        __syncthreads();
        for (int m = 0; m < 64; ++m) {
            float qa[4], kb[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { qa[a] = As[ty * 4 + a][m]; kb[a] = Bs[tx * 4 + a][m]; }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) pacc[a][b] = fmaf(qa[a], kb[b], pacc[a][b]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            Bs[i][j] = (j <= i && i < L) ? pacc[a][b] * dc_pow(la, i - j) : 0.f;
        }
    for (int idx = tid; idx < DC_C * 64; idx += 256) {
        const int j = idx >> 6, nn = idx & 63;
        float vv = 0.f;
        if (j < L && col0 + nn < p.dv) vv = siluf_(to_f32<T>(proj[(size_t)(t0 + j) * p.stride + p.v_off + h * p.dv + col0 + nn]));
        As[j][nn] = vv;
    }
    __syncthreads();
    // ---- O = P V
    float oacc[4][4] = {};
    for (int j = 0; j < L; ++j) {
        float pa[4], vb[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) { pa[a] = Bs[ty * 4 + a][j]; vb[a] = As[j][tx * 4 + a]; }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) oacc[a][b] = fmaf(pa[a], vb[b], oacc[a][b]);
    }
    // ---- O += diag(a^(i+1)) Q S, S the state before the chunk
    const float* S = p.U + ((size_t)chunk * p.heads + h) * p.dk * p.dv;
    for (int m0 = 0; m0 < p.dk; m0 += 64) {
        __syncthreads();
        for (int idx = tid; idx < DC_C * 64; idx += 256) {
            const int i = idx >> 6, m = idx & 63;
            float qv = 0.f;
            if (i < L && m0 + m < p.dk)
                qv = siluf_(to_f32<T>(proj[(size_t)(t0 + i) * p.stride + p.q_off + h * p.dk + m0 + m])) * dc_pow(la, i + 1);
            As[i][m] = qv;
            float sv = 0.f;                        // here i is the state's row within the slab, m its column
            if (m0 + i < p.dk && col0 + m < p.dv) sv = S[(size_t)(m0 + i) * p.dv + col0 + m];
            Bs[i][m] = sv;
        }
        __syncthreads();
        for (int m = 0; m < 64; ++m) {
            float qa[4], sb[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { qa[a] = As[ty * 4 + a][m]; sb[a] = Bs[m][tx * 4 + a]; }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) oacc[a][b] = fmaf(qa[a], sb[b], oacc[a][b]);
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = ty * 4 + a;
        if (i >= L) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int col = col0 + tx * 4 + b;
            if (col < p.dv) p.out[(size_t)(t0 + i) * p.heads * p.dv + h * p.dv + col] = oacc[a][b];
        }
    }
}

MSGL_API int msgl_decay_attention_chunked(const void* proj, long long stride, int q_off, int k_off, int v_off, int heads, int dk,
                                          int dv, const float* decay, float* state, const int* q_start, const int* slots,
                                          float* out, float* U, int n_chunks, int B, int dtype, cudaStream_t stream) {
    if (B <= 0 || n_chunks <= 0) return MSGL_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    DecayChunkParams p;
    p.proj = proj; p.stride = stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.heads = heads; p.dk = dk; p.dv = dv;
    p.B = B; p.decay = decay; p.state = state; p.q_start = q_start; p.slots = slots; p.U = U; p.out = out;
    const int n_rt = (dk + 63) / 64, n_ct = (dv + 63) / 64;
    if (dtype == MSGL_F32) decay_chunk_kv_kernel<float><<<dim3(n_chunks, heads, n_rt * n_ct), 256, 0, stream>>>(p);
    else decay_chunk_kv_kernel<__nv_bfloat16><<<dim3(n_chunks, heads, n_rt * n_ct), 256, 0, stream>>>(p);
    decay_chunk_scan_kernel<<<dim3(B, heads, (dk * dv + 255) / 256), 256, 0, stream>>>(p);
    if (dtype == MSGL_F32) decay_chunk_out_kernel<float><<<dim3(n_chunks, heads, n_ct), 256, 0, stream>>>(p);
    else decay_chunk_out_kernel<__nv_bfloat16><<<dim3(n_chunks, heads, n_ct), 256, 0, stream>>>(p);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// y = x / sqrt(mean(x^2) + eps) * w * sigmoid(gate) * c   (x float32 [T, N]; gate and y in packed rows)
// ---------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void rms_gate_kernel(const float* __restrict__ x, int N, const float* __restrict__ w, float eps, const void* gate_,
                                long long gate_stride, int gate_off, void* out_, long long out_stride, int out_off, float c) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * N;
    float ssq = 0.f;
    for (int i = threadIdx.x * V; i < N; i += blockDim.x * V) {
        float v[2];
        ld_v<V>(xr + i, v);
        ssq += v[0] * v[0] + v[1] * v[1];
    }
    ssq = block_sum(ssq, red);
    const float rs = 1.f / sqrtf(ssq / (float)N + eps);
    const T* g = gate_ ? reinterpret_cast<const T*>(gate_) + (size_t)t * gate_stride + gate_off : nullptr;
    T* o = reinterpret_cast<T*>(out_) + (size_t)t * out_stride + out_off;
    for (int i = threadIdx.x * V; i < N; i += blockDim.x * V) {
        float v[2], wv[2], gv[2] = {0.f, 0.f}, y[2];
        ld_v<V>(xr + i, v);
        ld_v<V>(w + i, wv);
        if (g) ld_v<V>(g + i, gv);
        y[0] = v[0] * rs * wv[0] * (g ? sigmoidf_(gv[0]) : 1.f) * c;
        y[1] = v[1] * rs * wv[1] * (g ? sigmoidf_(gv[1]) : 1.f) * c;
        st_v<V>(o + i, y);
    }
}

MSGL_API int msgl_rms_gate(const float* x, int N, const float* w, float eps, const void* gate, long long gate_stride, int gate_off,
                           void* out, long long out_stride, int out_off, float c, int T, int dtype, cudaStream_t stream) {
    if (T <= 0) return MSGL_OK;
    if (N <= 0) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const size_t item = dtype == MSGL_F32 ? 4 : 2;
    const bool v2 = even_all(N, gate_stride, gate_off, out_stride, out_off) && aligned_to(x, 8) && aligned_to(w, 8) &&
                    aligned_to(gate, 2 * item) && aligned_to(out, 2 * item);
    const int threads = N >= 2048 ? 512 : (N >= 512 ? 256 : 128);
    if (dtype == MSGL_F32) {
        if (v2) rms_gate_kernel<float, 2><<<T, threads, 0, stream>>>(x, N, w, eps, gate, gate_stride, gate_off, out, out_stride, out_off, c);
        else rms_gate_kernel<float, 1><<<T, threads, 0, stream>>>(x, N, w, eps, gate, gate_stride, gate_off, out, out_stride, out_off, c);
    } else {
        if (v2) rms_gate_kernel<__nv_bfloat16, 2><<<T, threads, 0, stream>>>(x, N, w, eps, gate, gate_stride, gate_off, out, out_stride, out_off, c);
        else rms_gate_kernel<__nv_bfloat16, 1><<<T, threads, 0, stream>>>(x, N, w, eps, gate, gate_stride, gate_off, out, out_stride, out_off, c);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out = act(gate) * up; act 0 = silu, 1 = gelu (tanh form), 2 = sigmoid
// ---------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void gated_act_kernel(const void* in_, long long in_stride, int gate_off, int up_off, void* out_, long long out_stride,
                                 int out_off, int I, int act) {
    const long long t = blockIdx.x;
    const T* in = reinterpret_cast<const T*>(in_) + t * in_stride;
    T* out = reinterpret_cast<T*>(out_) + t * out_stride + out_off;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * V; i < I; i += gridDim.y * blockDim.x * V) {
        float g[2], u[2], o[2];
        ld_v<V>(in + gate_off + i, g);
        ld_v<V>(in + up_off + i, u);
        o[0] = (act == 1 ? gelu_tanhf_(g[0]) : (act == 2 ? sigmoidf_(g[0]) : siluf_(g[0]))) * u[0];
        o[1] = V == 2 ? (act == 1 ? gelu_tanhf_(g[1]) : (act == 2 ? sigmoidf_(g[1]) : siluf_(g[1]))) * u[1] : 0.f;
        st_v<V>(out + i, o);
    }
}

MSGL_API int msgl_gated_act(const void* in, long long in_stride, int gate_off, int up_off, void* out, long long out_stride,
                            int out_off, int I, int act, int T, int dtype, cudaStream_t stream) {
    if (T <= 0 || I <= 0) return MSGL_OK;
    if (act < 0 || act > 2) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const size_t item = dtype == MSGL_F32 ? 4 : 2;
    const bool v2 = even_all(I, in_stride, gate_off, up_off, out_stride, out_off) && aligned_to(in, 2 * item) && aligned_to(out, 2 * item);
    const int per = v2 ? 2 : 1;
    const dim3 grid(T, max(1, min((I + 256 * per - 1) / (256 * per), 64)));
    if (dtype == MSGL_F32) {
        if (v2) gated_act_kernel<float, 2><<<grid, 256, 0, stream>>>(in, in_stride, gate_off, up_off, out, out_stride, out_off, I, act);
        else gated_act_kernel<float, 1><<<grid, 256, 0, stream>>>(in, in_stride, gate_off, up_off, out, out_stride, out_off, I, act);
    } else {
        if (v2) gated_act_kernel<__nv_bfloat16, 2><<<grid, 256, 0, stream>>>(in, in_stride, gate_off, up_off, out, out_stride, out_off, I, act);
        else gated_act_kernel<__nv_bfloat16, 1><<<grid, 256, 0, stream>>>(in, in_stride, gate_off, up_off, out, out_stride, out_off, I, act);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * c   (x dense [T, heads, d]; gate and out in packed rows)
// ---------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void head_gate_kernel(const T* __restrict__ x, const void* gate_, long long gate_stride, int gate_off, void* out_,
                                 long long out_stride, int out_off, int heads, int d, float c) {
    const long long t = blockIdx.x;
    const T* g = gate_ ? reinterpret_cast<const T*>(gate_) + t * gate_stride + gate_off : nullptr;
    T* o = reinterpret_cast<T*>(out_) + t * out_stride + out_off;
    const T* xr = x + t * heads * d;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * V; i < heads * d; i += gridDim.y * blockDim.x * V) {
        const float f = g ? sigmoidf_(to_f32<T>(g[i / d])) * c : c;       // d even: a pair lies within one head
        float v[2];
        ld_v<V>(xr + i, v);
        v[0] *= f; v[1] *= f;
        st_v<V>(o + i, v);
    }
}

MSGL_API int msgl_head_gate(const void* x, const void* gate, long long gate_stride, int gate_off, void* out, long long out_stride,
                            int out_off, int heads, int d, float c, int T, int dtype, cudaStream_t stream) {
    if (T <= 0) return MSGL_OK;
    if (heads <= 0 || d <= 0) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const size_t item = dtype == MSGL_F32 ? 4 : 2;
    const bool v2 = even_all(d, out_stride, out_off) && aligned_to(x, 2 * item) && aligned_to(out, 2 * item);
    const int per = v2 ? 2 : 1;
    const dim3 grid(T, max(1, min((heads * d + 256 * per - 1) / (256 * per), 16)));
    if (dtype == MSGL_F32) {
        if (v2) head_gate_kernel<float, 2><<<grid, 256, 0, stream>>>((const float*)x, gate, gate_stride, gate_off, out, out_stride, out_off, heads, d, c);
        else head_gate_kernel<float, 1><<<grid, 256, 0, stream>>>((const float*)x, gate, gate_stride, gate_off, out, out_stride, out_off, heads, d, c);
    } else {
        if (v2) head_gate_kernel<__nv_bfloat16, 2><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, gate, gate_stride, gate_off, out, out_stride, out_off, heads, d, c);
        else head_gate_kernel<__nv_bfloat16, 1><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, gate, gate_stride, gate_off, out, out_stride, out_off, heads, d, c);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// res[t, :] = float(E[ids[t], :]) * c: the float32 stream of a model that scales its embedding
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void scaled_embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                        int H, int V, float c) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    const bool ok = id >= 0 && id < V;               // the host validates ids; one out of range gives zeros, never a wild read
    const T* row = table + (size_t)(ok ? id : 0) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_f32<T>(row[i]) * c : 0.f;
}

MSGL_API int msgl_scaled_embedding(const int* ids, const void* table, float* out, int T_, int H, int V, float c, int dtype,
                                   cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0 || V <= 0) return MSGL_ERR_SIZE;
    const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
    if (dtype == MSGL_F32) scaled_embedding_kernel<float><<<T_, threads, 0, stream>>>(ids, (const float*)table, out, H, V, c);
    else if (dtype == MSGL_BF16)
        scaled_embedding_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, H, V, c);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// A sublayer's output normed before it joins the stream, and the next sublayer's input norm in the same pass:
//
//   res[t, :] += c * a[t, :] / sqrt(mean(a[t, :]^2) + eps_a) * w_a             (float32, in place)
//   y[t, :]    = res[t, :] / sqrt(mean(res[t, :]^2) + eps_y) * w_y             (only if w_y is given)
//
// One block per row; the row stays in registers between the passes (in shared memory beyond 8,192 columns).  a: activation
// type or float32.
// ---------------------------------------------------------------------------------------
template <typename T, typename A>
__global__ void postnorm_residual_kernel(const A* __restrict__ a, const float* __restrict__ w_a, float eps_a, float c,
                                         float* __restrict__ res, const float* __restrict__ w_y, float eps_y, T* __restrict__ y,
                                         int H) {
    extern __shared__ float prow[];                  // [H]
    __shared__ float red[32];
    const size_t off = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32<A>(a[off + i]);
        prow[i] = v;
        ss += v * v;
    }
    const float ra = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_a);
    ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {      // a thread reads back what it wrote itself
        const float v = res[off + i] + c * (prow[i] * ra * w_a[i]);
        res[off + i] = v;
        prow[i] = v;
        ss += v * v;
    }
    if (w_y == nullptr) return;
    const float ry = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_y);
    for (int i = threadIdx.x; i < H; i += blockDim.x) y[off + i] = from_f32<T>(prow[i] * ry * w_y[i]);
}

// The same with the row in registers (VPT values a thread, all loads of a row in flight together): rows up to 512 * VPT wide.
// Blocks of at most 512 threads, so that several rows share a multiprocessor and one row's sums overlap another's loads.
template <typename T, typename A, int VPT>
__global__ void __launch_bounds__(512) postnorm_residual_reg_kernel(const A* __restrict__ a, const float* __restrict__ w_a, float eps_a,
                                                                     float c, float* __restrict__ res, const float* __restrict__ w_y,
                                                                     float eps_y, T* __restrict__ y, int H) {
    __shared__ float red[32];
    const size_t off = (size_t)blockIdx.x * H;
    float av[VPT], rv[VPT], wa[VPT], wy[VPT];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const bool ok = i < H;
        av[k] = ok ? to_f32<A>(a[off + i]) : 0.f;
        rv[k] = ok ? res[off + i] : 0.f;
        wa[k] = ok ? w_a[i] : 0.f;
        wy[k] = (ok && w_y != nullptr) ? w_y[i] : 0.f;
        ss += av[k] * av[k];
    }
    const float ra = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_a);
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const float v = rv[k] + c * (av[k] * ra * wa[k]);
        if (i < H) res[off + i] = v;
        rv[k] = v;
        ss += v * v;
    }
    if (w_y == nullptr) return;
    const float ry = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_y);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < H) y[off + i] = from_f32<T>(rv[k] * ry * wy[k]);
    }
}

// The same with eight neighbouring columns a thread and access (16-byte loads and stores), G such groups a thread: rows whose
// width is a multiple of 8, up to 512 * 8 * G columns, every pointer 16-byte aligned.
template <typename T, typename A, int G>
__global__ void __launch_bounds__(512) postnorm_residual_vec_kernel(const A* __restrict__ a, const float* __restrict__ w_a, float eps_a,
                                                                    float c, float* __restrict__ res, const float* __restrict__ w_y,
                                                                    float eps_y, T* __restrict__ y, int H) {
    __shared__ float red[32];
    const size_t off = (size_t)blockIdx.x * H;
    float av[G][8], rv[G][8], wa[G][8], wy[G][8];
    float ss = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = (threadIdx.x + g * blockDim.x) * 8;
        if (i < H) {
            ld_w<8>(a + off + i, av[g]);
            ld_w<8>(res + off + i, rv[g]);
            ld_w<8>(w_a + i, wa[g]);
            if (w_y != nullptr) ld_w<8>(w_y + i, wy[g]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { av[g][e] = 0.f; rv[g][e] = 0.f; wa[g][e] = 0.f; }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += av[g][e] * av[g][e];
    }
    const float ra = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_a);
    ss = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = (threadIdx.x + g * blockDim.x) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v = rv[g][e] + c * (av[g][e] * ra * wa[g][e]);
            rv[g][e] = v;
            ss += v * v;
        }
        if (i < H) st_w<8>(res + off + i, rv[g]);
    }
    if (w_y == nullptr) return;
    const float ry = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps_y);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int i = (threadIdx.x + g * blockDim.x) * 8;
        if (i < H) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = rv[g][e] * ry * wy[g][e];
            st_w<8>(y + off + i, o);
        }
    }
}

MSGL_API int msgl_postnorm_residual(const void* a, int a_is_f32, const float* w_a, float eps_a, float c, float* res,
                                    const float* w_y, float eps_y, void* y, int rows, int H, int dtype, cudaStream_t stream) {
    if (rows <= 0) return MSGL_OK;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    if (H <= 8192 && H % 8 == 0 && aligned_to(a, 16) && aligned_to(res, 16) && aligned_to(w_a, 16) && aligned_to(w_y, 16) && aligned_to(y, 16)) {
        const int groups = H / 8;
        const int threads = min(512, (groups + 31) / 32 * 32);
        const bool two = groups > threads;
#define PNV_LAUNCH(T, A)                                                                                                       \
    do {                                                                                                                       \
        if (!two) postnorm_residual_vec_kernel<T, A, 1><<<rows, threads, 0, stream>>>((const A*)a, w_a, eps_a, c, res, w_y, eps_y, (T*)y, H); \
        else postnorm_residual_vec_kernel<T, A, 2><<<rows, threads, 0, stream>>>((const A*)a, w_a, eps_a, c, res, w_y, eps_y, (T*)y, H);      \
    } while (0)
        if (dtype == MSGL_F32) PNV_LAUNCH(float, float);
        else if (a_is_f32) PNV_LAUNCH(__nv_bfloat16, float);
        else PNV_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef PNV_LAUNCH
        return msgl_check_launch();
    }
    if (H <= 8192) {
        // the kernel and its block size follow from the row's width (and the buffers' alignment) alone, so a row's sums do not
        // depend on the batch
        const int vpt = H <= 4096 ? 8 : 16;
        const int threads = min(512, ((H + vpt - 1) / vpt + 31) / 32 * 32);
#define PNR_LAUNCH(T, A)                                                                                                       \
    do {                                                                                                                       \
        if (vpt == 8) postnorm_residual_reg_kernel<T, A, 8><<<rows, threads, 0, stream>>>((const A*)a, w_a, eps_a, c, res, w_y, eps_y, (T*)y, H); \
        else postnorm_residual_reg_kernel<T, A, 16><<<rows, threads, 0, stream>>>((const A*)a, w_a, eps_a, c, res, w_y, eps_y, (T*)y, H);         \
    } while (0)
        if (dtype == MSGL_F32) PNR_LAUNCH(float, float);
        else if (a_is_f32) PNR_LAUNCH(__nv_bfloat16, float);
        else PNR_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef PNR_LAUNCH
        return msgl_check_launch();
    }
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = 512;
#define PN_LAUNCH(T, A)                                                                                                    \
    do {                                                                                                                   \
        static MsglOncePerDevice once;                                                                                     \
        if (smem > 48 * 1024 && once.due()) {                                                                              \
            cudaFuncSetAttribute(postnorm_residual_kernel<T, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            once.mark();                                                                                                   \
        }                                                                                                                  \
        postnorm_residual_kernel<T, A><<<rows, threads, smem, stream>>>((const A*)a, w_a, eps_a, c, res, w_y, eps_y, (T*)y, H); \
    } while (0)
    if (dtype == MSGL_F32) PN_LAUNCH(float, float);
    else if (a_is_f32) PN_LAUNCH(__nv_bfloat16, float);
    else PN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef PN_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Latent attention, what a token leaves in the cache and the query latent:
//
//   proj row: the query's down-projection at column dq_off (q_rank wide; q_rank = 0: none), the key/value
//   down-projection at column dkv_off (kv_rank + rot_dim wide)
//   cq_out[t, :]               = rmsnorm(proj[dq ..]) * w_dq                                     (if q_rank > 0)
//   cache row [0, kv_rank)     = rmsnorm(proj[dkv .. dkv + kv_rank]) * w_dkv                     the latent
//   cache row [kv_rank, + rot_dim) = the last rot_dim columns, their first rot_dims rotated      one key part for all heads
//
// Rotation: element i < rot_dims / 2 with element i + rot_dims / 2, angle = position * freq[i] (float32), cos and sin times
// `mag`; elements from rot_dims on pass unchanged.  The cache has one kv head of size kv_rank + rot_dim:
// [page][slot in page][kv_rank + rot_dim].  One block per token.
// ---------------------------------------------------------------------------------------
struct LatentPrepParams {
    const void* proj; long long stride; int dq_off, dkv_off;
    int q_rank, kv_rank, rot_dim, rot_dims;
    const float* w_dq; const float* w_dkv; float eps;
    const float* freq; float mag;
    const int* positions; const int* out_loc;
    void* cq_out;                 // [T, q_rank]
    void* cache; int page_size;   // may be null: nothing is written to the cache
};

template <typename T>
__global__ void latent_prep_kernel(const LatentPrepParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const T* row = reinterpret_cast<const T*>(p.proj) + (size_t)t * p.stride;
    float sq = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) { const float v = to_f32<T>(row[p.dq_off + i]); sq += v * v; }
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) { const float v = to_f32<T>(row[p.dkv_off + i]); sc += v * v; }
    if (p.q_rank > 0) {
        const float rq = 1.f / sqrtf(block_sum(sq, red) / (float)p.q_rank + p.eps);
        T* cq = reinterpret_cast<T*>(p.cq_out) + (size_t)t * p.q_rank;
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) cq[i] = from_f32<T>(to_f32<T>(row[p.dq_off + i]) * rq * p.w_dq[i]);
    }
    const float rc = 1.f / sqrtf(block_sum(sc, red) / (float)p.kv_rank + p.eps);
    if (p.cache == nullptr) return;
    const int loc = p.out_loc[t];
    const int D = p.kv_rank + p.rot_dim;
    T* dst = reinterpret_cast<T*>(p.cache) + (size_t)loc * D;      // one kv head: token slot * row size
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(row[p.dkv_off + i]) * rc * p.w_dkv[i]);
    const T* kr = row + p.dkv_off + p.kv_rank;
    const int half = p.rot_dims / 2;
    const float pos = (float)p.positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * p.freq[i], &sn, &cs);
        sn *= p.mag; cs *= p.mag;
        const float u = to_f32<T>(kr[i]), v = to_f32<T>(kr[i + half]);
        dst[p.kv_rank + i] = from_f32<T>(u * cs - v * sn);
        dst[p.kv_rank + i + half] = from_f32<T>(v * cs + u * sn);
    }
    for (int i = p.rot_dims + threadIdx.x; i < p.rot_dim; i += blockDim.x) dst[p.kv_rank + i] = kr[i];
}

MSGL_API int msgl_latent_prep(const void* proj, long long stride, int dq_off, int dkv_off, int q_rank, int kv_rank, int rot_dim,
                              int rot_dims, const float* w_dq, const float* w_dkv, float eps, const float* freq, float mag,
                              const int* positions, const int* out_loc, void* cq_out, void* cache, int page_size, int T_,
                              int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1)) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    LatentPrepParams p;
    p.proj = proj; p.stride = stride; p.dq_off = dq_off; p.dkv_off = dkv_off; p.q_rank = q_rank; p.kv_rank = kv_rank;
    p.rot_dim = rot_dim; p.rot_dims = rot_dims; p.w_dq = w_dq; p.w_dkv = w_dkv; p.eps = eps; p.freq = freq; p.mag = mag;
    p.positions = positions; p.out_loc = out_loc; p.cq_out = cq_out; p.cache = cache; p.page_size = page_size;
    const int widest = max(q_rank, kv_rank);
    const int threads = widest >= 1024 ? 256 : (widest >= 256 ? 128 : 64);
    if (dtype == MSGL_F32) latent_prep_kernel<float><<<T_, threads, 0, stream>>>(p);
    else latent_prep_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(p);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The rotated part of every query head: src [T rows][heads][src_head] with the part at column src_off of a head, dst
// [T][heads][dst_head] with the part at column dst_off.  The first rot_dims of the part's rot_dim elements are rotated as
// above, the rest are copied.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_heads_kernel(const T* __restrict__ src, long long src_stride, int src_head, int src_off, T* __restrict__ dst,
                                  int dst_head, int dst_off, int heads, int rot_dim, int rot_dims,
                                  const float* __restrict__ freq, float mag, const int* __restrict__ positions) {
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    const T* s = src + (size_t)t * src_stride + src_off;
    T* d = dst + (size_t)t * heads * dst_head + dst_off;
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= mag; cs *= mag;
        const float u = to_f32<T>(s[(size_t)h * src_head + i]), v = to_f32<T>(s[(size_t)h * src_head + i + half]);
        d[(size_t)h * dst_head + i] = from_f32<T>(u * cs - v * sn);
        d[(size_t)h * dst_head + i + half] = from_f32<T>(v * cs + u * sn);
    }
    const int rest = rot_dim - rot_dims;
    for (int idx = threadIdx.x; idx < heads * rest; idx += blockDim.x) {
        const int h = idx / rest, i = rot_dims + idx - h * rest;
        d[(size_t)h * dst_head + i] = s[(size_t)h * src_head + i];
    }
}

MSGL_API int msgl_rope_heads(const void* src, long long src_stride, int src_head, int src_off, void* dst, int dst_head, int dst_off,
                             int heads, int rot_dim, int rot_dims, const float* freq, float mag, const int* positions, int T_,
                             int dtype, cudaStream_t stream) {
    if (T_ <= 0 || rot_dim == 0) return MSGL_OK;
    if (heads <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || src_off + rot_dim > src_head ||
        dst_off + rot_dim > dst_head)
        return MSGL_ERR_SIZE;
    const int work = heads * max(rot_dims / 2, rot_dim - rot_dims);
    const int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == MSGL_F32)
        rope_heads_kernel<float><<<T_, threads, 0, stream>>>((const float*)src, src_stride, src_head, src_off, (float*)dst, dst_head,
                                                             dst_off, heads, rot_dim, rot_dims, freq, mag, positions);
    else if (dtype == MSGL_BF16)
        rope_heads_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>((const __nv_bfloat16*)src, src_stride, src_head, src_off,
                                                                     (__nv_bfloat16*)dst, dst_head, dst_off, heads, rot_dim,
                                                                     rot_dims, freq, mag, positions);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out[t, i] = act(gate[t, i]) * x[t, i]; gate, x and out are [T, N] views into rows of their own strides; act 0 = silu,
// 2 = sigmoid
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ gate, long long gate_stride, const T* __restrict__ x, long long x_stride,
                                T* __restrict__ out, long long out_stride, int N, int act) {
    const long long t = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < N; i += gridDim.y * blockDim.x) {
        const float g = to_f32<T>(gate[t * gate_stride + i]);
        out[t * out_stride + i] = from_f32<T>((act == 2 ? sigmoidf_(g) : siluf_(g)) * to_f32<T>(x[t * x_stride + i]));
    }
}

MSGL_API int msgl_gate_mul(const void* gate, long long gate_stride, const void* x, long long x_stride, void* out,
                           long long out_stride, int N, int act, int T_, int dtype, cudaStream_t stream) {
    if (T_ <= 0 || N <= 0) return MSGL_OK;
    if (act != 0 && act != 2) return MSGL_ERR_SIZE;
    const dim3 grid(T_, max(1, min((N + 255) / 256, 32)));
    if (dtype == MSGL_F32)
        gate_mul_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate, gate_stride, (const float*)x, x_stride, (float*)out, out_stride, N, act);
    else if (dtype == MSGL_BF16)
        gate_mul_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gate, gate_stride, (const __nv_bfloat16*)x, x_stride,
                                                                 (__nv_bfloat16*)out, out_stride, N, act);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Linear attention whose decay comes from the input, per token and key channel:
//
//   q = proj q * q_scale, k = proj k [heads][dk], v = proj v [heads][dv]
//   alpha = sigmoid(z + bias)^(1 / tau) = exp(logsigmoid(z + bias) / tau), z float32 [T][heads * dk]
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  S per request [slot][heads][dk][dv] float32
//
// Same layout of the work as decay_attention_kernel: a block owns 32 columns of one (request, head) state and walks the
// request's tokens of the step in order.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float log_sigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int NR>
__global__ void __launch_bounds__(DA_COLS * DA_PARTS)
gated_decay_attention_kernel(const void* proj_, long long stride, int q_off, int k_off, int v_off, int heads, int dk, int dv,
                             const float* __restrict__ z, const float* __restrict__ z_bias, float inv_tau, float q_scale,
                             float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ slots,
                             float* __restrict__ out /* [T, heads * dv] */) {
    extern __shared__ float qka[];                   // [2][3][dk]: double-buffered q, k and decay of the current token
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DA_COLS;
    const int tid = threadIdx.x;
    const int part = tid & (DA_PARTS - 1), col = col0 + (tid >> 3);
    const bool col_ok = col < dv;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    const int slot = slots[r];
    const T* proj = reinterpret_cast<const T*>(proj_);
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    const int rows = (dk + DA_PARTS - 1) / DA_PARTS;             // rows i = part + DA_PARTS * j
    float s[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + DA_PARTS * j;
        s[j] = (j < rows && i < dk && col_ok) ? S[(size_t)i * dv + col] : 0.f;
    }
    for (int tt = 0; tt < n; ++tt) {
        const size_t row = (size_t)(t0 + tt) * stride;
        float* qb = qka + (tt & 1) * 3 * dk;
        float* kb = qb + dk;
        float* ab = kb + dk;
        for (int i = tid; i < dk; i += DA_COLS * DA_PARTS) {
            qb[i] = to_f32<T>(proj[row + q_off + h * dk + i]) * q_scale;
            kb[i] = to_f32<T>(proj[row + k_off + h * dk + i]);
            const float zz = z[(size_t)(t0 + tt) * heads * dk + h * dk + i] + z_bias[h * dk + i];
            ab[i] = expf(log_sigmoidf_(zz) * inv_tau);
        }
        const float v = col_ok ? to_f32<T>(proj[row + v_off + h * dv + col]) : 0.f;
        __syncthreads();
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            if (j < rows) {
                const int i = part + DA_PARTS * j;
                if (i < dk) {
                    s[j] = fmaf(ab[i], s[j], kb[i] * v);
                    acc = fmaf(s[j], qb[i], acc);
                }
            }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (part == 0 && col_ok) out[(size_t)(t0 + tt) * heads * dv + h * dv + col] = acc;
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + DA_PARTS * j;
        if (j < rows && i < dk && col_ok) S[(size_t)i * dv + col] = s[j];
    }
}

MSGL_API int msgl_gated_decay_attention(const void* proj, long long stride, int q_off, int k_off, int v_off, int heads, int dk,
                                        int dv, const float* z, const float* z_bias, float tau, float q_scale, float* state,
                                        const int* q_start, const int* slots, float* out, int B, int dtype, cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0 || dk > DA_PARTS * DA_MAX_ROWS || !(tau > 0.f)) return MSGL_ERR_SIZE;
    const dim3 grid(B, heads, (dv + DA_COLS - 1) / DA_COLS);
    const size_t smem = (size_t)6 * dk * sizeof(float);
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int nr = (dk + DA_PARTS - 1) / DA_PARTS;
    const float inv_tau = 1.f / tau;
#define GDA_LAUNCH(N)                                                                                                          \
    do {                                                                                                                       \
        if (dtype == MSGL_F32)                                                                                                 \
            gated_decay_attention_kernel<float, N><<<grid, DA_COLS * DA_PARTS, smem, stream>>>(                                \
                proj, stride, q_off, k_off, v_off, heads, dk, dv, z, z_bias, inv_tau, q_scale, state, q_start, slots, out);    \
        else                                                                                                                   \
            gated_decay_attention_kernel<__nv_bfloat16, N><<<grid, DA_COLS * DA_PARTS, smem, stream>>>(                        \
                proj, stride, q_off, k_off, v_off, heads, dk, dv, z, z_bias, inv_tau, q_scale, state, q_start, slots, out);    \
    } while (0)
    if (nr <= 4) GDA_LAUNCH(4);
    else if (nr <= 8) GDA_LAUNCH(8);
    else if (nr <= 16) GDA_LAUNCH(16);
    else if (nr <= 32) GDA_LAUNCH(32);
    else GDA_LAUNCH(64);
#undef GDA_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// y[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * w * act(gate[t, h, :]) * c
//   x float32 [T, heads, d] contiguous; w float32 [d], one weight for all heads; gate and y in packed rows;
//   act 0 = silu, 2 = sigmoid.  One warp per (token, head).
// ---------------------------------------------------------------------------------------
template <typename T, int NPL /* elements of a head per lane held in registers: head sizes up to 32 * NPL; 0: any size, two passes */>
__global__ void group_rms_gate_kernel(const float* __restrict__ x, int heads, int d, const float* __restrict__ w, float eps,
                                      const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride,
                                      float c, int act, long long n_rows) {
    const long long rowi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (rowi >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = rowi / heads;
    const int h = (int)(rowi - t * heads);
    const float* xr = x + rowi * d;
    const T* g = gate ? gate + t * gate_stride + (long long)h * d : nullptr;
    T* o = out + t * out_stride + (long long)h * d;
    if constexpr (NPL > 0) {
        float xv[NPL], gv[NPL], wv[NPL];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int i = lane + 32 * k;
            const bool ok = i < d;
            xv[k] = ok ? xr[i] : 0.f;
            gv[k] = (ok && g) ? to_f32<T>(g[i]) : 0.f;
            wv[k] = ok ? w[i] : 0.f;
            ss += xv[k] * xv[k];
        }
        const float rs = 1.f / sqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int i = lane + 32 * k;
            const float f = g ? c * (act == 2 ? sigmoidf_(gv[k]) : siluf_(gv[k])) : c;
            if (i < d) o[i] = from_f32<T>(xv[k] * rs * wv[k] * f);
        }
    } else {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = xr[i]; ss += v * v; }
        const float rs = 1.f / sqrtf(warp_sum(ss) / (float)d + eps);
        for (int i = lane; i < d; i += 32) {
            float f = c;
            if (g) { const float gv = to_f32<T>(g[i]); f *= (act == 2 ? sigmoidf_(gv) : siluf_(gv)); }
            o[i] = from_f32<T>(xr[i] * rs * w[i] * f);
        }
    }
}

MSGL_API int msgl_group_rms_gate(const float* x, int heads, int d, const float* w, float eps, const void* gate,
                                 long long gate_stride, void* out, long long out_stride, float c, int act, int T_, int dtype,
                                 cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (heads <= 0 || d <= 0 || (act != 0 && act != 2)) return MSGL_ERR_SIZE;
    const long long n_rows = (long long)T_ * heads;
    const int warps = 4;
    const unsigned blocks = (unsigned)((n_rows + warps - 1) / warps);
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
#define GRG_LAUNCH(N)                                                                                                          \
    do {                                                                                                                       \
        if (dtype == MSGL_F32)                                                                                                 \
            group_rms_gate_kernel<float, N><<<blocks, warps * 32, 0, stream>>>(x, heads, d, w, eps, (const float*)gate, gate_stride,   \
                                                                               (float*)out, out_stride, c, act, n_rows);       \
        else                                                                                                                   \
            group_rms_gate_kernel<__nv_bfloat16, N><<<blocks, warps * 32, 0, stream>>>(x, heads, d, w, eps, (const __nv_bfloat16*)gate, \
                                                                                       gate_stride, (__nv_bfloat16*)out, out_stride,    \
                                                                                       c, act, n_rows);                        \
    } while (0)
    if (d <= 128) GRG_LAUNCH(4);
    else if (d <= 256) GRG_LAUNCH(8);
    else if (d <= 512) GRG_LAUNCH(16);
    else GRG_LAUNCH(0);
#undef GRG_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The same gated linear attention for long portions: a request's tokens of the step in chunks of 64, the chunks in
// parallel.  With L tokens in a chunk (local index i), g_i = log2(alpha_i) per key channel, b_i = g_0 + ... + g_i, and S the
// state before the chunk:
//
//   1. gated_chunk_prep_kernel   b_i for every token (a running sum per channel within the chunk)
//   2. gated_chunk_kv_kernel     U = sum_i diag(2^(b_(L-1) - b_i)) k_i v_i^T                   every chunk by itself
//   3. gated_chunk_scan_kernel   per request, chunk after chunk: U <- S, S <- diag(2^b_(L-1)) S + U; the state row gets the last S
//   4. gated_chunk_p_kernel      P[i][j] = sum_c q_i[c] k_j[c] 2^(b_i[c] - b_j[c]) for j <= i, stored by key  (one exponential a term: every
//                                exponent is <= 0, so nothing overflows however strong the decay)
//   5. gated_chunk_out_kernel    o_i = (q_i * 2^b_i) S + sum_(j <= i) P[i][j] v_j
//
// All products are float32 FMA through shared memory (8 x 8 results a thread in the last kernel, 4 x 4 in the second, which
// was measured slower with the larger tile: its time goes into staging the decayed keys, not into the products); the results
// differ from the token-by-token kernel by rounding only.
// ---------------------------------------------------------------------------------------
struct GatedChunkParams {
    DecayChunkParams d;           // d.decay is not used
    const float* z; const float* z_bias; float inv_tau_log2e; float q_scale;
    float* bcum;                  // [T][heads * dk]
    float* P;                     // [chunks][heads][64 keys][64 queries]
};

__global__ void __launch_bounds__(128) gated_chunk_prep_kernel(const GatedChunkParams p) {
    __shared__ int sh[2];
    int req, t0, L;
    if (!dc_find_chunk(p.d, blockIdx.x, sh, req, t0, L)) return;
    const int HK = p.d.heads * p.d.dk;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (ch >= HK) return;
    const float bias = p.z_bias[ch];
    float run = 0.f;
    for (int i = 0; i < L; ++i) {
        const size_t at = (size_t)(t0 + i) * HK + ch;
        run += log_sigmoidf_(p.z[at] + bias) * p.inv_tau_log2e;
        p.bcum[at] = run;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) gated_chunk_kv_kernel(const GatedChunkParams p) {
    __shared__ __align__(16) float Ks[DC_C][64];
    __shared__ __align__(16) float Vs[DC_C][64];
    __shared__ int sh[2];
    const DecayChunkParams& d = p.d;
    const int chunk = blockIdx.x, h = blockIdx.y;
    const int n_ct = (d.dv + 63) / 64;
    const int row0 = (blockIdx.z / n_ct) * 64, col0 = (blockIdx.z % n_ct) * 64;
    int req, t0, L;
    if (!dc_find_chunk(d, chunk, sh, req, t0, L)) return;
    const int HK = d.heads * d.dk;
    const T* proj = reinterpret_cast<const T*>(d.proj);
    const int tid = threadIdx.x;
    for (int idx = tid; idx < DC_C * 64; idx += 256) {
        const int i = idx >> 6, m = idx & 63;
        float kv = 0.f, vv = 0.f;
        if (i < L) {
            const size_t row = (size_t)(t0 + i) * d.stride;
            if (row0 + m < d.dk) {
                const int ch = h * d.dk + row0 + m;
                const float e = p.bcum[(size_t)(t0 + L - 1) * HK + ch] - p.bcum[(size_t)(t0 + i) * HK + ch];
                kv = to_f32<T>(proj[row + d.k_off + ch]) * exp2f(fminf(e, 0.f));
            }
            if (col0 + m < d.dv) vv = to_f32<T>(proj[row + d.v_off + h * d.dv + col0 + m]);
        }
        Ks[i][m] = kv;
        Vs[i][m] = vv;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4] = {};
    for (int i = 0; i < L; ++i) {
        const float4 kr = *reinterpret_cast<const float4*>(&Ks[i][ty * 4]);
        const float4 vr = *reinterpret_cast<const float4*>(&Vs[i][tx * 4]);
        const float ka[4] = {kr.x, kr.y, kr.z, kr.w}, va[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ka[a], va[b], acc[a][b]);
    }
    float* U = d.U + ((size_t)chunk * d.heads + h) * d.dk * d.dv;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int row = row0 + ty * 4 + a;
        if (row >= d.dk) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int col = col0 + tx * 4 + b;
            if (col < d.dv) U[(size_t)row * d.dv + col] = acc[a][b];
        }
    }
}

__global__ void gated_chunk_scan_kernel(const GatedChunkParams p) {
    const DecayChunkParams& d = p.d;
    const int r = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int E = d.dk * d.dv;
    if (e >= E) return;
    const int base = d.q_start[r], n = d.q_start[r + 1] - base;
    if (n <= 0) return;
    int chunk0 = 0;
    for (int r2 = 0; r2 < r; ++r2) chunk0 += (d.q_start[r2 + 1] - d.q_start[r2] + DC_C - 1) / DC_C;
    const int HK = d.heads * d.dk;
    const int ch = h * d.dk + e / d.dv;
    float* st = d.state + ((size_t)d.slots[r] * d.heads + h) * E + e;
    float S = *st;
    const int nc = (n + DC_C - 1) / DC_C;
    // eight chunks at a time: their sums and decays are fetched together, then the state walks through them
    for (int c0 = 0; c0 < nc; c0 += 8) {
        float uv[8], f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;
            if (c < nc) {
                const int L = min(DC_C, n - c * DC_C);
                uv[k] = d.U[((size_t)(chunk0 + c) * d.heads + h) * E + e];
                f[k] = p.bcum[(size_t)(base + c * DC_C + L - 1) * HK + ch];
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;
            if (c < nc) {
                d.U[((size_t)(chunk0 + c) * d.heads + h) * E + e] = S;
                S = fmaf(exp2f(f[k]), S, uv[k]);
            }
        }
    }
    *st = S;
}

#define GC_IB 16        // rows of P a block makes
#define GC_CT 32        // key channels staged at a time
template <typename T>
__global__ void __launch_bounds__(256) gated_chunk_p_kernel(const GatedChunkParams p) {
    __shared__ float Qs[GC_IB][GC_CT + 1], BQs[GC_IB][GC_CT + 1];
    __shared__ float Ks[DC_C][GC_CT + 1], BKs[DC_C][GC_CT + 1];
    __shared__ int sh[2];
    const DecayChunkParams& d = p.d;
    const int chunk = blockIdx.x, h = blockIdx.y, ib = blockIdx.z;
    int req, t0, L;
    if (!dc_find_chunk(d, chunk, sh, req, t0, L)) return;
    float* P = p.P + ((size_t)chunk * d.heads + h) * DC_C * DC_C;
    const int tid = threadIdx.x, ii = tid >> 4, jj = tid & 15;
    const int i = ib * GC_IB + ii;
    if (ib * GC_IB >= L) {          // rows past the chunk's last token
        for (int m = 0; m < DC_C / 16; ++m) P[(size_t)(jj + 16 * m) * DC_C + i] = 0.f;
        return;
    }
    const int HK = d.heads * d.dk;
    const T* proj = reinterpret_cast<const T*>(d.proj);
    const int n_j = (ib + 1) * GC_IB;          // keys 0 .. n_j - 1 can be seen from this block's rows
    float acc[DC_C / 16] = {};
    for (int c0 = 0; c0 < d.dk; c0 += GC_CT) {
        __syncthreads();
        for (int idx = tid; idx < (GC_IB + n_j) * GC_CT; idx += 256) {
            const int rr = idx / GC_CT, c = idx - rr * GC_CT;
            const bool is_q = rr < GC_IB;
            const int tok = is_q ? ib * GC_IB + rr : rr - GC_IB;
            float x = 0.f, bb = 0.f;
            if (tok < L && c0 + c < d.dk) {
                const int ch = h * d.dk + c0 + c;
                x = to_f32<T>(proj[(size_t)(t0 + tok) * d.stride + (is_q ? d.q_off : d.k_off) + ch]);
                bb = p.bcum[(size_t)(t0 + tok) * HK + ch];
            }
            if (is_q) { Qs[rr][c] = x * p.q_scale; BQs[rr][c] = bb; }
            else { Ks[tok][c] = x; BKs[tok][c] = bb; }
        }
        __syncthreads();
        for (int c = 0; c < GC_CT; ++c) {
            const float qv = Qs[ii][c], bq = BQs[ii][c];
#pragma unroll
            for (int m = 0; m < DC_C / 16; ++m) {
                if (m <= ib) {
                    const int j = jj + 16 * m;
                    acc[m] = fmaf(qv * Ks[j][c], exp2f(fminf(bq - BKs[j][c], 0.f)), acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < DC_C / 16; ++m) {
        const int j = jj + 16 * m;
        P[(size_t)j * DC_C + i] = (m <= ib && j <= i && i < L) ? acc[m] : 0.f;          // stored by key: the next kernel sums over keys
    }
}

#define GO_TN 256       // output columns a block of gated_chunk_out_kernel makes
#define GO_LDA 68       // row length of the left operand's slabs: 16-byte rows, and a column's 64 stores spread over the banks
// 8 x 32 threads, 8 x 8 results a thread (tokens ty*4.. and 32+ty*4.., columns tx*4.. and 128+tx*4..).  Both products run over
// slabs of 64 of their inner index m, the left operand stored by m: the chunk's weights by key, then q * 2^b by key channel.
template <typename T>
__global__ void __launch_bounds__(256) gated_chunk_out_kernel(const GatedChunkParams p) {
    extern __shared__ __align__(16) float gsm[];
    float (*As)[GO_LDA] = reinterpret_cast<float (*)[GO_LDA]>(gsm);                  // [64 m][tokens]
    float (*Bs)[GO_TN] = reinterpret_cast<float (*)[GO_TN]>(gsm + DC_C * GO_LDA);    // [64 m][columns]
    __shared__ int sh[2];
    const DecayChunkParams& d = p.d;
    const int chunk = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GO_TN;
    int req, t0, L;
    if (!dc_find_chunk(d, chunk, sh, req, t0, L)) return;
    const int HK = d.heads * d.dk;
    const T* proj = reinterpret_cast<const T*>(d.proj);
    const int tid = threadIdx.x, ty = tid >> 5, tx = tid & 31;
    float acc[8][8] = {};
    auto products = [&](int n_m) {
        for (int m = 0; m < n_m; ++m) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[m][ty * 4]), a1 = *reinterpret_cast<const float4*>(&As[m][32 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[m][tx * 4]), b1 = *reinterpret_cast<const float4*>(&Bs[m][128 + tx * 4]);
            const float qa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, sb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(qa[a], sb[b], acc[a][b]);
        }
    };
    // ---- O = P V: the weights come stored by key
    const float* P = p.P + ((size_t)chunk * d.heads + h) * DC_C * DC_C;
    for (int idx = tid; idx < DC_C * DC_C; idx += 256) As[idx >> 6][idx & 63] = P[idx];
    for (int idx = tid; idx < DC_C * GO_TN; idx += 256) {
        const int j = idx / GO_TN, c = idx - j * GO_TN;
        float vv = 0.f;
        if (j < L && col0 + c < d.dv) vv = to_f32<T>(proj[(size_t)(t0 + j) * d.stride + d.v_off + h * d.dv + col0 + c]);
        Bs[j][c] = vv;
    }
    __syncthreads();
    products(L);
    // ---- O += (Q * 2^b) S, S the state before the chunk
    const float* S = d.U + ((size_t)chunk * d.heads + h) * d.dk * d.dv;
    for (int m0 = 0; m0 < d.dk; m0 += 64) {
        __syncthreads();
        for (int idx = tid; idx < DC_C * 64; idx += 256) {
            const int i = idx >> 6, m = idx & 63;            // token i, key channel m0 + m
            float qv = 0.f;
            if (i < L && m0 + m < d.dk) {
                const int ch = h * d.dk + m0 + m;
                qv = to_f32<T>(proj[(size_t)(t0 + i) * d.stride + d.q_off + ch]) * p.q_scale * exp2f(p.bcum[(size_t)(t0 + i) * HK + ch]);
            }
            As[m][i] = qv;
        }
        for (int idx = tid; idx < 64 * GO_TN; idx += 256) {
            const int m = idx / GO_TN, c = idx - m * GO_TN;
            float sv = 0.f;
            if (m0 + m < d.dk && col0 + c < d.dv) sv = S[(size_t)(m0 + m) * d.dv + col0 + c];
            Bs[m][c] = sv;
        }
        __syncthreads();
        products(min(64, d.dk - m0));
    }
#pragma unroll
    for (int a = 0; a < 8; ++a) {
        const int i = a < 4 ? ty * 4 + a : 32 + ty * 4 + a - 4;
        if (i >= L) continue;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int col = col0 + (b < 4 ? tx * 4 + b : 128 + tx * 4 + b - 4);
            if (col < d.dv) d.out[(size_t)(t0 + i) * d.heads * d.dv + h * d.dv + col] = acc[a][b];
        }
    }
}

MSGL_API int msgl_gated_decay_attention_chunked(const void* proj, long long stride, int q_off, int k_off, int v_off, int heads,
                                                int dk, int dv, const float* z, const float* z_bias, float tau, float q_scale,
                                                float* state, const int* q_start, const int* slots, float* out, float* U,
                                                float* bcum, float* P, int n_chunks, int B, int dtype, cudaStream_t stream) {
    if (B <= 0 || n_chunks <= 0) return MSGL_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f)) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    GatedChunkParams p;
    p.d.proj = proj; p.d.stride = stride; p.d.q_off = q_off; p.d.k_off = k_off; p.d.v_off = v_off; p.d.heads = heads; p.d.dk = dk;
    p.d.dv = dv; p.d.B = B; p.d.decay = nullptr; p.d.state = state; p.d.q_start = q_start; p.d.slots = slots; p.d.U = U; p.d.out = out;
    p.z = z; p.z_bias = z_bias; p.inv_tau_log2e = 1.4426950408889634f / tau; p.q_scale = q_scale; p.bcum = bcum; p.P = P;
    const int n_rt = (dk + 63) / 64, n_ct = (dv + 63) / 64, n_ot = (dv + GO_TN - 1) / GO_TN;
    const size_t smem_out = (size_t)DC_C * (GO_LDA + GO_TN) * sizeof(float);
    static MsglOncePerDevice once;
    if (once.due()) {
        cudaFuncSetAttribute(gated_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
        cudaFuncSetAttribute(gated_chunk_out_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
        once.mark();
    }
    gated_chunk_prep_kernel<<<dim3(n_chunks, (heads * dk + 127) / 128), 128, 0, stream>>>(p);
    if (dtype == MSGL_F32) gated_chunk_kv_kernel<float><<<dim3(n_chunks, heads, n_rt * n_ct), 256, 0, stream>>>(p);
    else gated_chunk_kv_kernel<__nv_bfloat16><<<dim3(n_chunks, heads, n_rt * n_ct), 256, 0, stream>>>(p);
    gated_chunk_scan_kernel<<<dim3(B, heads, (dk * dv + 255) / 256), 256, 0, stream>>>(p);
    if (dtype == MSGL_F32) gated_chunk_p_kernel<float><<<dim3(n_chunks, heads, DC_C / GC_IB), 256, 0, stream>>>(p);
    else gated_chunk_p_kernel<__nv_bfloat16><<<dim3(n_chunks, heads, DC_C / GC_IB), 256, 0, stream>>>(p);
    if (dtype == MSGL_F32) gated_chunk_out_kernel<float><<<dim3(n_chunks, heads, n_ot), 256, smem_out, stream>>>(p);
    else gated_chunk_out_kernel<__nv_bfloat16><<<dim3(n_chunks, heads, n_ot), 256, smem_out, stream>>>(p);
    return msgl_check_launch();
}
