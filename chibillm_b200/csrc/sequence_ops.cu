// Kernels of the parts that carry a fixed-size state from token to token, and
// the small row-wise kernels around them:
//
// * short_conv: y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j) per channel, with the
//   inputs before a step's first token taken from the request's history;
// * delta_rule: the recurrence S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r with one
//   state matrix per head, decays, rates and unit keys made in 32-bit from the
//   stacked product's output;
// * gated_group_norm: x / rms(x per group) * weight * sigmoid(gate);
// * scale, cast_rows, add_row_vector, activation.
//
// Everything that enters the recurrence, and the state itself, is 32-bit in the
// bfloat16 engine too.
#define CHIBI_UNIT sequence_ops
#define CHIBI_UNIT_ID 7
#include "common.cuh"

namespace chibi {

// ---------------------------------------------------------------- short convolution
// grid (channel blocks, chunks of a sequence's tokens, sequences).  A thread owns one
// channel of one chunk of CONV_CHUNK consecutive tokens of one sequence.  Only the
// first chunk of a sequence reads the history (a chunk is at least taps - 1 tokens
// long), and the same thread writes the new history after its last read, so nobody
// reads a history that another thread has replaced.
template <typename TX>
__global__ void __launch_bounds__(128)
short_conv_kernel(const TX* __restrict__ x, long long x_stride, const float* __restrict__ w, TX* history,
                  TX* __restrict__ out, long long out_stride, const int* __restrict__ q_start,
                  const int* __restrict__ slots, int channels, int taps, int chunk)
{
    pdl_enter();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.z;
    const int row0 = q_start[seq];
    const int q_len = q_start[seq + 1] - row0;
    const int first = blockIdx.y * chunk;
    if (ch >= channels || first >= q_len)
        return;
    const int keep = taps - 1;
    const int last = min(first + chunk, q_len);
    TX* hist = history + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    const float* wc = w + (size_t)ch * taps;
    for (int i = first; i < last; ++i) {
        float y = to_f32(x[(size_t)(row0 + i) * x_stride + ch]);
        for (int j = 0; j < taps; ++j) {
            const int m = i - keep + j;                    // token of the sequence's step, or before it
            const float v = m >= 0 ? to_f32(x[(size_t)(row0 + m) * x_stride + ch])
                                   : to_f32(hist[(size_t)(keep + m) * channels + ch]);
            y = fmaf(wc[j], v, y);
        }
        out[(size_t)(row0 + i) * out_stride + ch] = from_f32<TX>(y);
    }
    if (first == 0) {
        // new history = the last `keep` entries of [old history ; this step's inputs], oldest first;
        // entry m is read from further along than it is written to, so ascending order is safe
        for (int m = 0; m < keep; ++m) {
            const int at = q_len + m;                      // index into the joined sequence
            hist[(size_t)m * channels + ch] = at < keep ? hist[(size_t)at * channels + ch]
                                                        : x[(size_t)(row0 + at - keep) * x_stride + ch];
        }
    }
}

// ---------------------------------------------------------------- delta rule
constexpr int DELTA_LANES = 8;        // threads that share a value column (its key rows in equal parts)
constexpr int DELTA_COLS = 16;        // value columns per CTA
constexpr int DELTA_THREADS = DELTA_LANES * DELTA_COLS;

struct DeltaParams {
    const void* proj;                 // [T, stride]: r | k | v | gate | removal | low, heads * d each but low
    long long stride;
    const float* decay_out;           // [rank, heads * d]: transposed, so that a warp's channels lie side by side
    const float* decay_logits;        // [T, heads * d] = tanh(low) decay_out, made by a matrix product before
                                      // this kernel (many tokens), or null: the kernel adds them up itself
    const float* decay_bias;          // [heads * d]
    const float* removal_bias;        // [heads * d]
    float* state;                     // [slots, heads, d (value), d (key)]
    float* o;                         // [T, heads * d]
    const int* q_start;
    const int* slots;
    int heads, d, rank, chunk;
    int late_trigger;                 // several chunks: the kernel after this one is let in only at the end
    float decay_scale, key_eps;
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// grid (column blocks, heads, sequences).  R: key rows per thread (a thread owns rows
// lane * R .. lane * R + R - 1 of its column; rows beyond d are zeros).  The sequence's
// tokens are taken in chunks: first all threads turn the chunk's projections into the
// five vectors of each token (decay, rate * unit key, unit key, key, receptance; a warp
// per token), then every thread runs the recurrence over the chunk on its part of the
// state, which stays in registers from the sequence's first token of the step to its last.
//
// A sequence of many tokens keeps its CTAs busy for milliseconds.  The kernel that follows must not
// be let in at the start, as the short kernels do it: its CTAs would sit on the SMs waiting and
// take issue slots from the recurrence (a prompt of 2,048 tokens took 38 ms instead of 6).  With
// several chunks the kernel therefore triggers its dependents after the last token.
template <int R, typename TX>
__global__ void __launch_bounds__(DELTA_THREADS) delta_rule_kernel(const DeltaParams p)
{
#ifdef CHIBI_TIMELINE
    pdl_enter();
#else
    if (!p.late_trigger)
        pdl_trigger();
    pdl_wait();
#endif
    extern __shared__ __align__(16) float smem[];
    constexpr int DP = R * DELTA_LANES;                     // padded head size
    const int d = p.d, W = p.heads * d;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int col0 = blockIdx.x * DELTA_COLS;
    const int row0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - row0;
    if (q_len <= 0)
        return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cc = threadIdx.x / DELTA_LANES, part = threadIdx.x % DELTA_LANES;
    const int col = col0 + cc;
    const bool col_ok = col < d;
    // shared: per token of the chunk [decay | rate * u | u | k | r] (DP each), then v (DELTA_COLS),
    // then tanh(low) (rank)
    const int per_token = 5 * DP + DELTA_COLS + ((p.rank + 3) & ~3);      // a multiple of four floats
    const TX* proj = static_cast<const TX*>(p.proj);

    float S[R];
    float* st = p.state + (((size_t)p.slots[seq] * p.heads + head) * d + (col_ok ? col : 0)) * d;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
        S[i] = (col_ok && row < d) ? st[row] : 0.f;
    }

    for (int base = 0; base < q_len; base += p.chunk) {
        const int n = min(p.chunk, q_len - base);
        __syncthreads();                                    // the chunk before has been used up
        for (int tt = warp; tt < n; tt += DELTA_THREADS / 32) {
            float* v5 = smem + (size_t)tt * per_token;
            float* low = v5 + 5 * DP + DELTA_COLS;
            const TX* row = proj + (size_t)(row0 + base + tt) * p.stride;
            if (!p.decay_logits)
                for (int j = lane; j < p.rank; j += 32)
                    low[j] = tanhf(to_f32(row[5 * (size_t)W + j]));
            float ksq = 0.f;
            for (int c = lane; c < d; c += 32) {
                const float k = to_f32(row[W + head * d + c]);
                ksq = fmaf(k, k, ksq);
            }
            ksq = warp_sum(ksq);
            __syncwarp();
            const float inv = 1.f / sqrtf(ksq + p.key_eps);
            for (int c = lane; c < DP; c += 32) {
                float decay = 0.f, au = 0.f, u = 0.f, k = 0.f, r = 0.f;
                if (c < d) {
                    const int f = head * d + c;
                    float z = 0.f;
                    if (p.decay_logits) {
                        z = p.decay_logits[(size_t)(row0 + base + tt) * W + f];
                    } else {
                        const float* wcol = p.decay_out + f;
#pragma unroll 8
                        for (int j = 0; j < p.rank; ++j)
                            z = fmaf(wcol[(size_t)j * W], low[j], z);
                    }
                    decay = expf(-p.decay_scale * sigmoidf_(z + p.decay_bias[f]));
                    k = to_f32(row[W + f]);
                    r = to_f32(row[f]);
                    u = k * inv;
                    au = sigmoidf_(to_f32(row[4 * (size_t)W + f]) + p.removal_bias[f]) * u;
                }
                v5[c] = decay;
                v5[DP + c] = au;
                v5[2 * DP + c] = u;
                v5[3 * DP + c] = k;
                v5[4 * DP + c] = r;
            }
            if (lane < DELTA_COLS)
                v5[5 * DP + lane] = col0 + lane < d ? to_f32(row[2 * (size_t)W + head * d + col0 + lane]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float* v5 = smem + (size_t)tt * per_token + part * R;
            const float v = smem[(size_t)tt * per_token + 5 * DP + cc];
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 u = *reinterpret_cast<const float4*>(v5 + 2 * DP + i);
                dot = fmaf(u.x, S[i], dot);
                dot = fmaf(u.y, S[i + 1], dot);
                dot = fmaf(u.z, S[i + 2], dot);
                dot = fmaf(u.w, S[i + 3], dot);
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 w = *reinterpret_cast<const float4*>(v5 + i);
                const float4 au = *reinterpret_cast<const float4*>(v5 + DP + i);
                const float4 k = *reinterpret_cast<const float4*>(v5 + 3 * DP + i);
                const float4 r = *reinterpret_cast<const float4*>(v5 + 4 * DP + i);
                S[i] = fmaf(k.x, v, fmaf(w.x, S[i], -au.x * dot));
                S[i + 1] = fmaf(k.y, v, fmaf(w.y, S[i + 1], -au.y * dot));
                S[i + 2] = fmaf(k.z, v, fmaf(w.z, S[i + 2], -au.z * dot));
                S[i + 3] = fmaf(k.w, v, fmaf(w.w, S[i + 3], -au.w * dot));
                acc = fmaf(S[i], r.x, acc);
                acc = fmaf(S[i + 1], r.y, acc);
                acc = fmaf(S[i + 2], r.z, acc);
                acc = fmaf(S[i + 3], r.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (part == 0 && col_ok)
                p.o[(size_t)(row0 + base + tt) * W + head * d + col] = acc;
        }
    }
#ifndef CHIBI_TIMELINE
    if (p.late_trigger)
        pdl_trigger();
#endif
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
        if (col_ok && row < d)
            st[row] = S[i];
    }
}

// ---------------------------------------------------------------- gated group norm
// One warp per (row, group): out = x / sqrt(mean(x^2 over the group) + eps) * weight * sigmoid(gate).
template <typename TG, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ x, const TG* __restrict__ gate,
                                        long long gate_stride, const float* __restrict__ weight,
                                        TO* __restrict__ out, long long rows, int groups, int n, float eps)
{
    pdl_enter();
    const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (job >= rows * groups)
        return;
    const long long row = job / groups;
    const int g = (int)(job - row * groups);
    const float* src = x + ((size_t)row * groups + g) * n;
    float s = 0.f;
    for (int j = lane; j < n; j += 32)
        s = fmaf(src[j], src[j], s);
    s = warp_sum(s);
    const float inv = 1.f / sqrtf(s / (float)n + eps);
    const TG* gr = gate + (size_t)row * gate_stride + (size_t)g * n;
    TO* dst = out + ((size_t)row * groups + g) * n;
    for (int j = lane; j < n; j += 32)
        dst[j] = from_f32<TO>(src[j] * inv * weight[g * n + j] * sigmoidf_(to_f32(gr[j])));
}

// ---------------------------------------------------------------- row-wise helpers
__global__ void scale_kernel(float* __restrict__ x, float factor, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] *= factor;
}

template <typename TX, typename TO>
__global__ void cast_rows_kernel(const TX* __restrict__ x, long long x_stride, TO* __restrict__ out,
                                 long long out_stride, long long rows, int n, int act)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        const float v = to_f32(x[(size_t)r * x_stride + c]);
        out[(size_t)r * out_stride + c] = from_f32<TO>(act >= 0 ? activate(v, act) : v);
    }
}

__global__ void add_row_vector_kernel(float* __restrict__ acc, long long stride, const float* __restrict__ vec,
                                      long long rows, int n)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        acc[(size_t)r * stride + c] += vec[c];
    }
}

template <typename TX>
__global__ void activation_kernel(TX* __restrict__ x, long long total, int kind)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f32<TX>(activate(to_f32(x[i]), kind));
}

// out = act(sum over the splits of a split product's partial sums [splits][total])
template <typename TO>
__global__ void reduce_activation_kernel(const float* __restrict__ partial, int splits, long long total,
                                         TO* __restrict__ out, int kind)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float s = partial[i];
        for (int sp = 1; sp < splits; ++sp)
            s += partial[(size_t)sp * total + i];
        out[i] = from_f32<TO>(activate(s, kind));
    }
}

static int blocks_for(long long total, int block)
{
    long long b = (total + block - 1) / block;
    const long long cap = 148LL * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_short_conv(const void* x, int x_type, long long x_stride, const float* w, void* history,
                               void* out, long long out_stride, const int* q_start, const int* slots, int seqs,
                               int max_q_len, int channels, int taps, cudaStream_t stream)
{
    if (seqs <= 0 || max_q_len <= 0)
        return CHIBI_OK;
    if (channels <= 0 || taps < 1)
        return CHIBI_ERR_ARGUMENT;
    const int chunk = taps - 1 > 16 ? taps - 1 : 16;
    const long long chunks = ((long long)max_q_len + chunk - 1) / chunk;
    if (chunks > 65535 || seqs > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)((channels + 127) / 128), (unsigned)chunks, (unsigned)seqs);
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(short_conv_kernel<TX>, grid, dim3(128), 0, stream, (const TX*)x, x_stride, w, (TX*)history, (TX*)out,
               out_stride, q_start, slots, channels, taps, chunk);
    });
    return launch_status();
}

template <int R, typename TX>
static int launch_delta(const DeltaParams& p, int seqs, int max_q_len, cudaStream_t stream)
{
    constexpr int DP = R * DELTA_LANES;
    const int per_token = 5 * DP + DELTA_COLS + ((p.rank + 3) & ~3);
    int chunk = (int)((46 * 1024) / (per_token * sizeof(float)));
    if (chunk < 1)
        return CHIBI_ERR_UNSUPPORTED;
    chunk = chunk > 16 ? 16 : chunk;
    chunk = chunk > max_q_len ? max_q_len : chunk;
    DeltaParams q = p;
    q.chunk = chunk;
    q.late_trigger = max_q_len > chunk ? 1 : 0;
    const dim3 grid((unsigned)((p.d + DELTA_COLS - 1) / DELTA_COLS), (unsigned)p.heads, (unsigned)seqs);
    launch(delta_rule_kernel<R, TX>, grid, dim3(DELTA_THREADS), (size_t)chunk * per_token * sizeof(float), stream, q);
    return launch_status();
}

CHIBI_API int chibi_delta_rule(const void* proj, int x_type, long long stride, const float* decay_out,
                               const float* decay_logits, const float* decay_bias, const float* removal_bias, float* state, float* o,
                               const int* q_start, const int* slots, int seqs, int max_q_len, int heads, int d,
                               int rank, float decay_scale, float key_eps, cudaStream_t stream)
{
    if (seqs <= 0 || max_q_len <= 0)
        return CHIBI_OK;
    if (heads <= 0 || d <= 0 || rank <= 0 || (!decay_out && !decay_logits))
        return CHIBI_ERR_ARGUMENT;
    if (d > 256 || heads > 65535 || seqs > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    DeltaParams p = { proj, stride, decay_out, decay_logits, decay_bias, removal_bias, state, o, q_start, slots,
                      heads, d, rank, 0, 0, decay_scale, key_eps };
    const int rows = (d + DELTA_LANES - 1) / DELTA_LANES;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        if (rows <= 4)
            return launch_delta<4, TX>(p, seqs, max_q_len, stream);
        if (rows <= 8)
            return launch_delta<8, TX>(p, seqs, max_q_len, stream);
        if (rows <= 12)
            return launch_delta<12, TX>(p, seqs, max_q_len, stream);
        if (rows <= 16)
            return launch_delta<16, TX>(p, seqs, max_q_len, stream);
        if (rows <= 24)
            return launch_delta<24, TX>(p, seqs, max_q_len, stream);
        return launch_delta<32, TX>(p, seqs, max_q_len, stream);
    });
    return CHIBI_OK;
}

CHIBI_API int chibi_gated_group_norm(const float* x, const void* gate, int gate_type, long long gate_stride,
                                     const float* weight, void* out, int out_type, long long rows, int groups,
                                     int n, float eps, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (groups <= 0 || n <= 0)
        return CHIBI_ERR_ARGUMENT;
    const long long jobs = rows * groups;
    const long long blocks = (jobs + 3) / 4;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(gate_type, TG, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(gated_group_norm_kernel<TG, TO>, dim3((unsigned)blocks), dim3(128), 0, stream, x, (const TG*)gate,
               gate_stride, weight, (TO*)out, rows, groups, n, eps);
    }));
    return launch_status();
}

CHIBI_API int chibi_scale(float* x, float factor, long long total, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    launch(scale_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, stream, x, factor, total);
    return launch_status();
}

// `act`: -1 none, else the activation by that code is applied on the way.
CHIBI_API int chibi_cast_rows(const void* x, int x_type, long long x_stride, void* out, int out_type,
                              long long out_stride, long long rows, int n, int act, cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    if (act < -1 || act > 4)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(cast_rows_kernel<TX, TO>, dim3(blocks_for(rows * n, 256)), dim3(256), 0, stream, (const TX*)x, x_stride,
               (TO*)out, out_stride, rows, n, act);
    }));
    return launch_status();
}

CHIBI_API int chibi_add_row_vector(float* acc, long long stride, const float* vec, long long rows, int n,
                                   cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    launch(add_row_vector_kernel, dim3(blocks_for(rows * n, 256)), dim3(256), 0, stream, acc, stride, vec, rows, n);
    return launch_status();
}

CHIBI_API int chibi_activation(void* x, int x_type, long long total, int kind, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (kind < 0 || kind > 4)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(activation_kernel<TX>, dim3(blocks_for(total, 256)), dim3(256), 0, stream, (TX*)x, total, kind);
    });
    return launch_status();
}

CHIBI_API int chibi_reduce_activation(const float* partial, int splits, long long total, void* out, int out_type,
                                      int kind, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (kind < 0 || kind > 4 || splits < 1)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(reduce_activation_kernel<TO>, dim3(blocks_for(total, 256)), dim3(256), 0, stream, partial, splits, total,
               (TO*)out, kind);
    });
    return launch_status();
}
