// Tensor-core attention for any sequence length (warp-level mma.sync
// m16n8k8, TF32 operands rounded to nearest, FP32 accumulation).
//
// Same contract as the FP32 kernels in attention.cu (reference
// src/ops.c:1297-1355 and :1381-1441): head-major Q, K, V, O, the full
// probability matrix P is written by the forward pass and read by the
// backward pass.  Work decomposition: one block of four warps per
// (group, tile of 64 rows); a warp owns 16 rows; the other axis is swept in
// tiles of 64 staged in shared memory.
//
//   forward    sweep 1: S = scale Q K^T, running row maximum and denominator
//              sweep 2: S again, P = exp(S - max) / denominator -> global,
//                       O += P V
//   backward   D_i = dO_i . O_i
//              query-major: dP = dO V^T, dS = scale P (dP - D), dQ (+)= dS K
//              key-major:   dS recomputed,  dK (+)= dS^T Q,  dV (+)= P^T dO
//
// Tiles are stored in shared memory already rounded to TF32.  Tile pitches
// are chosen so that fragment loads are bank-conflict free in the layout each
// tile is read most.
#include "kernels.h"
#include "device_util.cuh"

#include <cfloat>

namespace vitb200 {
namespace {

constexpr int kRows = 64;        // rows per block, and per sweep tile
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kScorePitch = 72;  // [64][64] score tiles: 72 = 8 (mod 32)

__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ void mma_16x8x8(float (&c)[4], const float (&a)[4],
                                           float b0, float b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])),
          "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
          "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// Fragment coordinates of this lane: g = row within 8, t = column within 4.
struct Lane {
    int g, t;
    __device__ Lane() : g((threadIdx.x & 31) >> 2), t(threadIdx.x & 3) {}
};

// A fragment (16 x 8) of a row-major tile: rows row0..row0+15, columns k0..k0+7.
__device__ __forceinline__ void load_a(float (&a)[4], const float *tile,
                                       int pitch, int row0, int k0,
                                       const Lane &lane) {
    const float *p = tile + (row0 + lane.g) * pitch + k0 + lane.t;
    a[0] = p[0];
    a[1] = p[8 * pitch];
    a[2] = p[4];
    a[3] = p[8 * pitch + 4];
}

// A fragment of the transpose of a row-major tile: A(r, k) = tile[k0+k][row0+r].
__device__ __forceinline__ void load_a_transposed(float (&a)[4],
                                                  const float *tile, int pitch,
                                                  int row0, int k0,
                                                  const Lane &lane) {
    const float *p = tile + (k0 + lane.t) * pitch + row0 + lane.g;
    a[0] = p[0];
    a[1] = p[8];
    a[2] = p[4 * pitch];
    a[3] = p[4 * pitch + 8];
}

// C[16 x 8*NB] += A * B with B(k, n) = tile_b[n0 + n][k]  ("rows are n").
template <int NB>
__device__ __forceinline__ void gemm_b_rows_n(float (&c)[NB][4],
                                              const float *tile_a, int pitch_a,
                                              int row0, const float *tile_b,
                                              int pitch_b, int n0, int depth,
                                              const Lane &lane) {
    for (int k0 = 0; k0 < depth; k0 += 8) {
        float a[4];
        load_a(a, tile_a, pitch_a, row0, k0, lane);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const float *p = tile_b + (n0 + nb * 8 + lane.g) * pitch_b + k0 + lane.t;
            mma_16x8x8(c[nb], a, p[0], p[4]);
        }
    }
}

// C[16 x 8*NB] += A * B with B(k, n) = tile_b[k][n0 + n]  ("rows are k");
// A comes from `tile_a`, read directly or transposed.
template <int NB, bool kTransposedA>
__device__ __forceinline__ void gemm_b_rows_k(float (&c)[NB][4],
                                              const float *tile_a, int pitch_a,
                                              int row0, const float *tile_b,
                                              int pitch_b, int n0, int depth,
                                              const Lane &lane) {
    for (int k0 = 0; k0 < depth; k0 += 8) {
        float a[4];
        if (kTransposedA) {
            load_a_transposed(a, tile_a, pitch_a, row0, k0, lane);
        } else {
            load_a(a, tile_a, pitch_a, row0, k0, lane);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const float *p = tile_b + (k0 + lane.t) * pitch_b + n0 + nb * 8 + lane.g;
            mma_16x8x8(c[nb], a, p[0], p[4 * pitch_b]);
        }
    }
}

// Stages rows [row0, row0+64) of a [seq, HD] matrix, rounded to TF32; rows
// past `seq` are zero.
template <int HD>
__device__ __forceinline__ void stage_rows(const float *__restrict__ source,
                                           float *tile, int row0, int seq) {
    constexpr int kPitch = HD + 4;
    constexpr int kVectors = HD / 4;
    for (int i = threadIdx.x; i < kRows * kVectors; i += kThreads) {
        const int r = i / kVectors;
        const int c = (i % kVectors) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < seq) {
            v = *reinterpret_cast<const float4 *>(source + size_t(row0 + r) * HD + c);
        }
        float *p = tile + r * kPitch + c;
        p[0] = round_tf32(v.x);
        p[1] = round_tf32(v.y);
        p[2] = round_tf32(v.z);
        p[3] = round_tf32(v.w);
    }
}

template <int NB>
__device__ __forceinline__ void clear(float (&c)[NB][4]) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.0f;
    }
}

// Sum / max over the four lanes that share a fragment row.
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
    return fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(kFullMask, v, 1);
    return v + __shfl_xor_sync(kFullMask, v, 2);
}

// ------------------------------------------------------------------ forward

template <int HD>
__global__ void __launch_bounds__(kThreads)
attention_mma_forward_kernel(const float *__restrict__ q,
                             const float *__restrict__ k,
                             const float *__restrict__ v, float *__restrict__ p,
                             float *__restrict__ out, int seq, float scale) {
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *q_tile = shared;                      // [64][HD+4]
    float *kv_tile = q_tile + kRows * kPitch;    // [64][HD+4]
    float *p_tile = kv_tile + kRows * kPitch;    // [64][72]
    const Lane lane;
    const int warp = threadIdx.x >> 5;
    const int row0 = warp * 16;                  // this warp's rows in the tile
    const size_t group = blockIdx.x;
    const int query0 = blockIdx.y * kRows;
    const size_t base = group * size_t(seq) * HD;

    stage_rows<HD>(q + base, q_tile, query0, seq);

    // Sweep 1: running maximum and denominator of the two rows this lane sees
    // (fragment rows g and g + 8).
    float maximum[2] = {-FLT_MAX, -FLT_MAX};
    float denominator[2] = {0.0f, 0.0f};
    for (int key0 = 0; key0 < seq; key0 += kRows) {
        __syncthreads();
        stage_rows<HD>(k + base, kv_tile, key0, seq);
        __syncthreads();
        float s[8][4];
        clear<8>(s);
        gemm_b_rows_n<8>(s, q_tile, kPitch, row0, kv_tile, kPitch, 0, HD, lane);
        float tile_max[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nb * 8 + 2 * lane.t + (e & 1);
                s[nb][e] = key < seq ? s[nb][e] * scale : -FLT_MAX;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[nb][e]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float updated = fmaxf(maximum[h], quad_max(tile_max[h]));
            float sum = 0.0f;
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
                sum += __expf(s[nb][2 * h] - updated) +
                       __expf(s[nb][2 * h + 1] - updated);
            }
            denominator[h] = denominator[h] * __expf(maximum[h] - updated) +
                             quad_sum(sum);
            maximum[h] = updated;
        }
    }
    const float inverse[2] = {1.0f / denominator[0], 1.0f / denominator[1]};

    // Sweep 2: probabilities to global memory, O += P V.
    float o[HD / 8][4];
    clear<HD / 8>(o);
    float *p_group = p + group * size_t(seq) * seq;
    for (int key0 = 0; key0 < seq; key0 += kRows) {
        __syncthreads();
        stage_rows<HD>(k + base, kv_tile, key0, seq);
        __syncthreads();
        float s[8][4];
        clear<8>(s);
        gemm_b_rows_n<8>(s, q_tile, kPitch, row0, kv_tile, kPitch, 0, HD, lane);
        __syncthreads();   // everyone is done with K before V replaces it
        stage_rows<HD>(v + base, kv_tile, key0, seq);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int col = nb * 8 + 2 * lane.t + (e & 1);
                const float probability = key0 + col < seq
                    ? __expf(s[nb][e] * scale - maximum[h]) * inverse[h]
                    : 0.0f;
                p_tile[(row0 + lane.g + 8 * h) * kScorePitch + col] = probability;
            }
        }
        __syncthreads();
        // Coalesced copy of the block's probability tile to global memory.
        for (int i = threadIdx.x; i < kRows * kRows; i += kThreads) {
            const int r = i >> 6, c = i & 63;
            if (query0 + r < seq && key0 + c < seq) {
                p_group[size_t(query0 + r) * seq + key0 + c] =
                    p_tile[r * kScorePitch + c];
            }
        }
        // The MMA reads the same tile; TF32 rounding happens in the tensor
        // core (low mantissa bits are ignored), which is harmless for values
        // in [0, 1].
        gemm_b_rows_k<HD / 8, false>(o, p_tile, kScorePitch, row0, kv_tile,
                                     kPitch, 0, kRows, lane);
    }
#pragma unroll
    for (int nb = 0; nb < HD / 8; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = query0 + row0 + lane.g + 8 * h;
            if (row < seq && out != nullptr) {
                *reinterpret_cast<float2 *>(out + base + size_t(row) * HD +
                                            nb * 8 + 2 * lane.t) =
                    make_float2(o[nb][2 * h], o[nb][2 * h + 1]);
            }
        }
    }
}

// ----------------------------------------------------------------- backward

// Loads the [64 x 64] block of the group's probability matrix whose top-left
// corner is (row0, col0) into a shared tile; out-of-range entries are zero.
__device__ __forceinline__ void stage_probabilities(
    const float *__restrict__ p_group, float *tile, int row0, int col0,
    int seq) {
    for (int i = threadIdx.x; i < kRows * kRows; i += kThreads) {
        const int r = i >> 6, c = i & 63;
        tile[r * kScorePitch + c] =
            (row0 + r < seq && col0 + c < seq)
                ? __ldcs(p_group + size_t(row0 + r) * seq + col0 + c)
                : 0.0f;
    }
}

// Writes (or adds) a warp's [16 x HD] accumulator to rows of a [seq, HD] matrix.
template <int HD>
__device__ __forceinline__ void store_rows(float *__restrict__ target,
                                           const float (&c)[HD / 8][4],
                                           int first_row, int seq, bool add,
                                           const Lane &lane) {
#pragma unroll
    for (int nb = 0; nb < HD / 8; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = first_row + lane.g + 8 * h;
            if (row < seq) {
                float2 *t = reinterpret_cast<float2 *>(
                    target + size_t(row) * HD + nb * 8 + 2 * lane.t);
                float2 value = add ? *t : make_float2(0.f, 0.f);
                value.x += c[nb][2 * h];
                value.y += c[nb][2 * h + 1];
                *t = value;
            }
        }
    }
}

// Forward pass that never forms P in memory: one sweep over the keys with a
// running row maximum and denominator, the output rescaled as the maximum
// grows.  Saves the row log-sum-exp so the backward pass can rebuild any
// probability as exp(scale s_ij - lse_i).
template <int HD>
__global__ void __launch_bounds__(kThreads)
attention_mma_flash_forward_kernel(const float *__restrict__ q,
                                   const float *__restrict__ k,
                                   const float *__restrict__ v,
                                   float *__restrict__ out,
                                   float *__restrict__ lse, int seq,
                                   float scale) {
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *q_tile = shared;
    float *k_tile = q_tile + kRows * kPitch;
    float *v_tile = k_tile + kRows * kPitch;
    float *p_tile = v_tile + kRows * kPitch;     // [64][72], rows private to a warp
    const Lane lane;
    const int row0 = (threadIdx.x >> 5) * 16;
    const size_t group = blockIdx.x;
    const int query0 = blockIdx.y * kRows;
    const size_t base = group * size_t(seq) * HD;

    stage_rows<HD>(q + base, q_tile, query0, seq);
    float maximum[2] = {-FLT_MAX, -FLT_MAX};
    float denominator[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
    clear<HD / 8>(o);
    for (int key0 = 0; key0 < seq; key0 += kRows) {
        __syncthreads();
        stage_rows<HD>(k + base, k_tile, key0, seq);
        stage_rows<HD>(v + base, v_tile, key0, seq);
        __syncthreads();
        float s[8][4];
        clear<8>(s);
        gemm_b_rows_n<8>(s, q_tile, kPitch, row0, k_tile, kPitch, 0, HD, lane);
        float tile_max[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nb * 8 + 2 * lane.t + (e & 1);
                s[nb][e] = key < seq ? s[nb][e] * scale : -FLT_MAX;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[nb][e]);
            }
        }
        float correction[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float updated = fmaxf(maximum[h], quad_max(tile_max[h]));
            correction[h] = __expf(maximum[h] - updated);
            maximum[h] = updated;
            float sum = 0.0f;
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
                s[nb][2 * h] = __expf(s[nb][2 * h] - updated);
                s[nb][2 * h + 1] = __expf(s[nb][2 * h + 1] - updated);
                sum += s[nb][2 * h] + s[nb][2 * h + 1];
            }
            denominator[h] = denominator[h] * correction[h] + quad_sum(sum);
        }
#pragma unroll
        for (int nb = 0; nb < HD / 8; ++nb) {
            o[nb][0] *= correction[0];
            o[nb][1] *= correction[0];
            o[nb][2] *= correction[1];
            o[nb][3] *= correction[1];
        }
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p_tile[(row0 + lane.g + 8 * (e >> 1)) * kScorePitch + nb * 8 +
                       2 * lane.t + (e & 1)] = s[nb][e];
            }
        }
        __syncwarp();
        gemm_b_rows_k<HD / 8, false>(o, p_tile, kScorePitch, row0, v_tile,
                                     kPitch, 0, kRows, lane);
        __syncwarp();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float inverse = 1.0f / denominator[h];
#pragma unroll
        for (int nb = 0; nb < HD / 8; ++nb) {
            o[nb][2 * h] *= inverse;
            o[nb][2 * h + 1] *= inverse;
        }
        const int row = query0 + row0 + lane.g + 8 * h;
        if (lane.t == 0 && row < seq) {
            lse[group * seq + row] = maximum[h] + __logf(denominator[h]);
        }
    }
    store_rows<HD>(out + base, o, query0 + row0, seq, false, lane);
}

template <int HD, bool kRecompute>
__global__ void __launch_bounds__(kThreads)
attention_mma_backward_query_kernel(const float *__restrict__ q,
                                    const float *__restrict__ k,
                                    const float *__restrict__ v,
                                    const float *__restrict__ p,
                                    const float *__restrict__ lse,
                                    const float *__restrict__ dout,
                                    const float *__restrict__ row_dots,
                                    float *__restrict__ dq, int seq,
                                    float scale, bool add_q) {
    // kRecompute: P is not read from memory but rebuilt per tile as
    // exp(scale Q K^T - lse); `p` is unused then, `q` and `lse` otherwise.
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *do_tile = shared;
    float *k_tile = do_tile + kRows * kPitch;
    float *v_tile = k_tile + kRows * kPitch;
    float *s_tile = v_tile + kRows * kPitch;     // P, then dS, [64][72]
    float *q_tile = s_tile + kRows * kScorePitch;  // only with kRecompute
    const Lane lane;
    const int warp = threadIdx.x >> 5;
    const int row0 = warp * 16;
    const size_t group = blockIdx.x;
    const int query0 = blockIdx.y * kRows;
    const size_t base = group * size_t(seq) * HD;
    const float *p_group = p + group * size_t(seq) * seq;

    stage_rows<HD>(dout + base, do_tile, query0, seq);
    if (kRecompute) {
        stage_rows<HD>(q + base, q_tile, query0, seq);
    }
    float dot[2], row_lse[2];
    bool row_live[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = query0 + row0 + lane.g + 8 * h;
        row_live[h] = row < seq;
        dot[h] = row_live[h] ? row_dots[group * seq + row] : 0.0f;
        row_lse[h] = (kRecompute && row_live[h]) ? lse[group * seq + row] : 0.0f;
    }
    float acc[HD / 8][4];
    clear<HD / 8>(acc);
    for (int key0 = 0; key0 < seq; key0 += kRows) {
        __syncthreads();
        stage_rows<HD>(k + base, k_tile, key0, seq);
        stage_rows<HD>(v + base, v_tile, key0, seq);
        if (!kRecompute) {
            stage_probabilities(p_group, s_tile, query0, key0, seq);
        }
        __syncthreads();
        if (kRecompute) {
            float s[8][4];
            clear<8>(s);
            gemm_b_rows_n<8>(s, q_tile, kPitch, row0, k_tile, kPitch, 0, HD, lane);
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int col = nb * 8 + 2 * lane.t + (e & 1);
                    s_tile[(row0 + lane.g + 8 * h) * kScorePitch + col] =
                        (row_live[h] && key0 + col < seq)
                            ? __expf(s[nb][e] * scale - row_lse[h]) : 0.0f;
                }
            }
        }
        float dp[8][4];
        clear<8>(dp);
        gemm_b_rows_n<8>(dp, do_tile, kPitch, row0, v_tile, kPitch, 0, HD, lane);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                float *cell = s_tile + (row0 + lane.g + 8 * h) * kScorePitch +
                              nb * 8 + 2 * lane.t + (e & 1);
                *cell = scale * *cell * (dp[nb][e] - dot[h]);
            }
        }
        __syncwarp();
        gemm_b_rows_k<HD / 8, false>(acc, s_tile, kScorePitch, row0, k_tile,
                                     kPitch, 0, kRows, lane);
    }
    store_rows<HD>(dq + base, acc, query0 + row0, seq, add_q, lane);
}

template <int HD, bool kRecompute>
__global__ void __launch_bounds__(kThreads)
attention_mma_backward_key_kernel(const float *__restrict__ q,
                                  const float *__restrict__ k,
                                  const float *__restrict__ v,
                                  const float *__restrict__ p,
                                  const float *__restrict__ lse,
                                  const float *__restrict__ dout,
                                  const float *__restrict__ row_dots,
                                  float *__restrict__ dk, float *__restrict__ dv,
                                  int seq, float scale, bool add_k,
                                  bool add_v) {
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *v_own = shared;                       // this block's 64 keys
    float *q_tile = v_own + kRows * kPitch;      // current 64 queries
    float *do_tile = q_tile + kRows * kPitch;
    float *p_tile = do_tile + kRows * kPitch;    // [query][key], pitch 72
    float *s_tile = p_tile + kRows * kScorePitch;
    float *dots = s_tile + kRows * kScorePitch;  // [64]
    float *lses = dots + kRows;                  // [64], only with kRecompute
    float *k_own = lses + kRows;                 // [64][HD+4], only with kRecompute
    const Lane lane;
    const int warp = threadIdx.x >> 5;
    const int row0 = warp * 16;
    const size_t group = blockIdx.x;
    const int key0 = blockIdx.y * kRows;
    const size_t base = group * size_t(seq) * HD;
    const float *p_group = p + group * size_t(seq) * seq;

    stage_rows<HD>(v + base, v_own, key0, seq);
    if (kRecompute) {
        stage_rows<HD>(k + base, k_own, key0, seq);
    }
    float acc_k[HD / 8][4], acc_v[HD / 8][4];
    clear<HD / 8>(acc_k);
    clear<HD / 8>(acc_v);
    for (int query0 = 0; query0 < seq; query0 += kRows) {
        __syncthreads();
        stage_rows<HD>(q + base, q_tile, query0, seq);
        stage_rows<HD>(dout + base, do_tile, query0, seq);
        if (!kRecompute) {
            stage_probabilities(p_group, p_tile, query0, key0, seq);
        }
        if (threadIdx.x < kRows) {
            const bool live = query0 + threadIdx.x < seq;
            dots[threadIdx.x] =
                live ? row_dots[group * seq + query0 + threadIdx.x] : 0.0f;
            if (kRecompute) {
                lses[threadIdx.x] =
                    live ? lse[group * seq + query0 + threadIdx.x] : 0.0f;
            }
        }
        __syncthreads();
        if (kRecompute) {
            // P for query rows row0..row0+15 against this block's 64 keys.
            float s[8][4];
            clear<8>(s);
            gemm_b_rows_n<8>(s, q_tile, kPitch, row0, k_own, kPitch, 0, HD, lane);
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = row0 + lane.g + 8 * (e >> 1);
                    const int c = nb * 8 + 2 * lane.t + (e & 1);
                    p_tile[r * kScorePitch + c] =
                        (query0 + r < seq && key0 + c < seq)
                            ? __expf(s[nb][e] * scale - lses[r]) : 0.0f;
                }
            }
            __syncwarp();
        }
        // Score gradients of query rows row0..row0+15 against all 64 keys.
        float dp[8][4];
        clear<8>(dp);
        gemm_b_rows_n<8>(dp, do_tile, kPitch, row0, v_own, kPitch, 0, HD, lane);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = row0 + lane.g + 8 * (e >> 1);
                const int c = nb * 8 + 2 * lane.t + (e & 1);
                s_tile[r * kScorePitch + c] =
                    scale * p_tile[r * kScorePitch + c] * (dp[nb][e] - dots[r]);
            }
        }
        __syncthreads();
        // This warp's 16 keys: dK += dS^T Q, dV += P^T dO over the 64 queries.
        gemm_b_rows_k<HD / 8, true>(acc_k, s_tile, kScorePitch, row0, q_tile,
                                    kPitch, 0, kRows, lane);
        gemm_b_rows_k<HD / 8, true>(acc_v, p_tile, kScorePitch, row0, do_tile,
                                    kPitch, 0, kRows, lane);
    }
    store_rows<HD>(dk + base, acc_k, key0 + row0, seq, add_k, lane);
    store_rows<HD>(dv + base, acc_v, key0 + row0, seq, add_v, lane);
}

__global__ void mma_row_dots_kernel(const float *__restrict__ a,
                                    const float *__restrict__ b,
                                    float *__restrict__ out, size_t rows,
                                    int head_dim) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const size_t warps = (size_t(gridDim.x) * blockDim.x) >> 5;
    for (size_t row = warp; row < rows; row += warps) {
        float sum = 0.0f;
        for (int d = lane; d < head_dim; d += 32) {
            sum += a[row * head_dim + d] * b[row * head_dim + d];
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            out[row] = sum;
        }
    }
}

// ------------------------------------------------- whole group in one tile
//
// For seq <= 64 the whole (sample, head) group fits one 64-row tile, so each
// pass needs a single sweep: scores stay in registers between the product and
// the softmax, and the backward pass computes dQ, dK and dV from one staging
// of Q, K, V, dO and P.

// Plain 128-bit copy of a [seq, HD] matrix into a 64-row tile (rows past seq
// are zero); rounding to TF32 is left to the tensor core, which ignores the
// low mantissa bits.
template <int HD>
__device__ __forceinline__ void stage_rows_raw(const float *__restrict__ source,
                                               float *tile, int seq) {
    constexpr int kPitch = HD + 4;
    constexpr int kVectors = HD / 4;
    for (int i = threadIdx.x; i < kRows * kVectors; i += kThreads) {
        const int r = i / kVectors;
        const int c = (i % kVectors) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < seq) {
            v = __ldcs(reinterpret_cast<const float4 *>(source + size_t(r) * HD + c));
        }
        *reinterpret_cast<float4 *>(tile + r * kPitch + c) = v;
    }
}

template <int HD>
__global__ void __launch_bounds__(kThreads)
attention_mma_single_forward_kernel(const float *__restrict__ q,
                                    const float *__restrict__ k,
                                    const float *__restrict__ v,
                                    float *__restrict__ p,
                                    float *__restrict__ out, int seq,
                                    float scale) {
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *q_tile = shared;
    float *k_tile = q_tile + kRows * kPitch;
    float *v_tile = k_tile + kRows * kPitch;
    float *p_tile = v_tile + kRows * kPitch;
    const Lane lane;
    const int row0 = (threadIdx.x >> 5) * 16;
    const size_t group = blockIdx.x;
    const size_t base = group * size_t(seq) * HD;
    stage_rows_raw<HD>(q + base, q_tile, seq);
    stage_rows_raw<HD>(k + base, k_tile, seq);
    stage_rows_raw<HD>(v + base, v_tile, seq);
    __syncthreads();
    float s[8][4];
    clear<8>(s);
    gemm_b_rows_n<8>(s, q_tile, kPitch, row0, k_tile, kPitch, 0, HD, lane);
    float maximum[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = nb * 8 + 2 * lane.t + (e & 1);
            s[nb][e] = key < seq ? s[nb][e] * scale : -FLT_MAX;
            maximum[e >> 1] = fmaxf(maximum[e >> 1], s[nb][e]);
        }
    }
    float inverse[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        maximum[h] = quad_max(maximum[h]);
        float sum = 0.0f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            s[nb][2 * h] = __expf(s[nb][2 * h] - maximum[h]);
            s[nb][2 * h + 1] = __expf(s[nb][2 * h + 1] - maximum[h]);
            sum += s[nb][2 * h] + s[nb][2 * h + 1];
        }
        inverse[h] = 1.0f / quad_sum(sum);
    }
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p_tile[(row0 + lane.g + 8 * (e >> 1)) * kScorePitch + nb * 8 +
                   2 * lane.t + (e & 1)] = s[nb][e] * inverse[e >> 1];
        }
    }
    __syncwarp();
    // Each warp writes its own 16 rows of P (contiguous in global memory).
    float *p_group = p + group * size_t(seq) * seq;
    for (int r = row0; r < row0 + 16 && r < seq; ++r) {
        for (int c = threadIdx.x & 31; c < seq; c += 32) {
            p_group[r * seq + c] = p_tile[r * kScorePitch + c];
        }
    }
    float o[HD / 8][4];
    clear<HD / 8>(o);
    gemm_b_rows_k<HD / 8, false>(o, p_tile, kScorePitch, row0, v_tile, kPitch,
                                 0, kRows, lane);
    store_rows<HD>(out + base, o, row0, seq, false, lane);
}

template <int HD>
__global__ void __launch_bounds__(kThreads)
attention_mma_single_backward_kernel(
    const float *__restrict__ q, const float *__restrict__ k,
    const float *__restrict__ v, const float *__restrict__ p,
    const float *__restrict__ out, const float *__restrict__ dout,
    float *__restrict__ dq, float *__restrict__ dk, float *__restrict__ dv,
    int seq, float scale, bool add_q, bool add_k, bool add_v) {
    constexpr int kPitch = HD + 4;
    extern __shared__ __align__(16) float shared[];
    float *q_tile = shared;
    float *k_tile = q_tile + kRows * kPitch;
    float *v_tile = k_tile + kRows * kPitch;
    float *do_tile = v_tile + kRows * kPitch;
    float *p_tile = do_tile + kRows * kPitch;
    float *s_tile = p_tile + kRows * kScorePitch;
    const Lane lane;
    const int row0 = (threadIdx.x >> 5) * 16;
    const size_t group = blockIdx.x;
    const size_t base = group * size_t(seq) * HD;
    stage_rows_raw<HD>(q + base, q_tile, seq);
    stage_rows_raw<HD>(k + base, k_tile, seq);
    stage_rows_raw<HD>(v + base, v_tile, seq);
    stage_rows_raw<HD>(dout + base, do_tile, seq);
    stage_probabilities(p + group * size_t(seq) * seq, p_tile, 0, 0, seq);
    // D_i = dO_i . O_i for the two fragment rows of this lane: the four lanes
    // of a quad split the row.
    float dot[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + lane.g + 8 * h;
        float sum = 0.0f;
        if (row < seq) {
            for (int d = lane.t * 4; d < HD; d += 16) {
                const float4 a = __ldcs(reinterpret_cast<const float4 *>(
                    out + base + size_t(row) * HD + d));
                const float4 b = __ldcs(reinterpret_cast<const float4 *>(
                    dout + base + size_t(row) * HD + d));
                sum += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
            }
        }
        dot[h] = quad_sum(sum);
    }
    __syncthreads();
    float dp[8][4];
    clear<8>(dp);
    gemm_b_rows_n<8>(dp, do_tile, kPitch, row0, v_tile, kPitch, 0, HD, lane);
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int cell = (row0 + lane.g + 8 * (e >> 1)) * kScorePitch +
                             nb * 8 + 2 * lane.t + (e & 1);
            s_tile[cell] = scale * p_tile[cell] * (dp[nb][e] - dot[e >> 1]);
        }
    }
    __syncthreads();
    float acc[HD / 8][4];
    clear<HD / 8>(acc);
    gemm_b_rows_k<HD / 8, false>(acc, s_tile, kScorePitch, row0, k_tile, kPitch,
                                 0, kRows, lane);
    store_rows<HD>(dq + base, acc, row0, seq, add_q, lane);
    clear<HD / 8>(acc);
    gemm_b_rows_k<HD / 8, true>(acc, s_tile, kScorePitch, row0, q_tile, kPitch,
                                0, kRows, lane);
    store_rows<HD>(dk + base, acc, row0, seq, add_k, lane);
    clear<HD / 8>(acc);
    gemm_b_rows_k<HD / 8, true>(acc, p_tile, kScorePitch, row0, do_tile, kPitch,
                                0, kRows, lane);
    store_rows<HD>(dv + base, acc, row0, seq, add_v, lane);
}

template <typename Kernel>
bool allow(Kernel kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        return cudaFuncSetAttribute(kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(bytes)) == cudaSuccess;
    }
    return true;
}

}  // namespace

bool attention_mma_supported(size_t head_dim) {
    return head_dim == 8 || head_dim == 16 || head_dim == 32 ||
           head_dim == 64 || head_dim == 128;
}

#define VITB200_MMA_DISPATCH(head_dim, CALL)                                   \
    switch (head_dim) {                                                        \
        case 8: CALL(8); break;                                                \
        case 16: CALL(16); break;                                              \
        case 32: CALL(32); break;                                              \
        case 64: CALL(64); break;                                              \
        default: CALL(128); break;                                             \
    }

bool launch_attention_mma_forward(const float *q, const float *k,
                                  const float *v, float *probabilities,
                                  float *out, size_t groups, size_t seq,
                                  size_t head_dim, float scale,
                                  cudaStream_t stream) {
    const dim3 grid(unsigned(groups), unsigned((seq + kRows - 1) / kRows));
    const size_t bytes =
        (2 * kRows * (head_dim + 4) + kRows * kScorePitch) * sizeof(float);
    bool launched = false;
    if (seq <= size_t(kRows) && head_dim <= 64) {
        const size_t single =
            (3 * kRows * (head_dim + 4) + kRows * kScorePitch) * sizeof(float);
#define CALL(HD)                                                               \
    if (allow(attention_mma_single_forward_kernel<HD>, single)) {              \
        attention_mma_single_forward_kernel<HD>                                \
            <<<unsigned(groups), kThreads, single, stream>>>(                  \
                q, k, v, probabilities, out, int(seq), scale);                 \
        launched = true;                                                       \
    }
        VITB200_MMA_DISPATCH(head_dim, CALL)
#undef CALL
        g_kernel_launches += launched ? 1 : 0;
        return launched;
    }
#define CALL(HD)                                                               \
    if (allow(attention_mma_forward_kernel<HD>, bytes)) {                      \
        attention_mma_forward_kernel<HD><<<grid, kThreads, bytes, stream>>>(   \
            q, k, v, probabilities, out, int(seq), scale);                     \
        launched = true;                                                       \
    }
    VITB200_MMA_DISPATCH(head_dim, CALL)
#undef CALL
    g_kernel_launches += launched ? 1 : 0;
    return launched;
}

bool launch_attention_mma_flash_forward(const float *q, const float *k,
                                        const float *v, float *out, float *lse,
                                        size_t groups, size_t seq,
                                        size_t head_dim, float scale,
                                        cudaStream_t stream) {
    const dim3 grid(unsigned(groups), unsigned((seq + kRows - 1) / kRows));
    const size_t bytes =
        (3 * kRows * (head_dim + 4) + kRows * kScorePitch) * sizeof(float);
    bool launched = false;
#define CALL(HD)                                                               \
    if (allow(attention_mma_flash_forward_kernel<HD>, bytes)) {                \
        attention_mma_flash_forward_kernel<HD>                                 \
            <<<grid, kThreads, bytes, stream>>>(q, k, v, out, lse, int(seq),   \
                                                scale);                        \
        launched = true;                                                       \
    }
    VITB200_MMA_DISPATCH(head_dim, CALL)
#undef CALL
    g_kernel_launches += launched ? 1 : 0;
    return launched;
}

bool launch_attention_mma_backward(const float *q, const float *k,
                                   const float *v, const float *probabilities,
                                   const float *lse, const float *out,
                                   const float *dout, float *dq, float *dk,
                                   float *dv, float *row_dots, size_t groups,
                                   size_t seq, size_t head_dim, float scale,
                                   bool add_q, bool add_k, bool add_v,
                                   cudaStream_t stream) {
    // lse != nullptr: probabilities are rebuilt from Q, K and the saved row
    // log-sum-exp instead of being read.
    const bool recompute = lse != nullptr;
    const dim3 grid(unsigned(groups), unsigned((seq + kRows - 1) / kRows));
    const size_t tile = kRows * (head_dim + 4);
    const size_t query_bytes =
        ((recompute ? 4 : 3) * tile + kRows * kScorePitch) * sizeof(float);
    const size_t key_bytes =
        ((recompute ? 4 : 3) * tile + 2 * kRows * kScorePitch + 2 * kRows) *
        sizeof(float);
    bool launched = false;
    if (!recompute && seq <= size_t(kRows) && head_dim <= 64) {
        const size_t single =
            (4 * tile + 2 * kRows * kScorePitch) * sizeof(float);
#define CALL(HD)                                                               \
    if (allow(attention_mma_single_backward_kernel<HD>, single)) {             \
        attention_mma_single_backward_kernel<HD>                               \
            <<<unsigned(groups), kThreads, single, stream>>>(                  \
                q, k, v, probabilities, out, dout, dq, dk, dv, int(seq),       \
                scale, add_q, add_k, add_v);                                   \
        launched = true;                                                       \
    }
        VITB200_MMA_DISPATCH(head_dim, CALL)
#undef CALL
        g_kernel_launches += launched ? 1 : 0;
        return launched;
    }
#define LAUNCH(HD, RECOMPUTE)                                                  \
    if (allow(attention_mma_backward_query_kernel<HD, RECOMPUTE>, query_bytes) && \
        allow(attention_mma_backward_key_kernel<HD, RECOMPUTE>, key_bytes)) {  \
        mma_row_dots_kernel<<<stream_grid(groups * seq * 32), kStreamThreads,  \
                              0, stream>>>(dout, out, row_dots, groups * seq,  \
                                           int(head_dim));                     \
        attention_mma_backward_query_kernel<HD, RECOMPUTE>                     \
            <<<grid, kThreads, query_bytes, stream>>>(                         \
                q, k, v, probabilities, lse, dout, row_dots, dq, int(seq),     \
                scale, add_q);                                                 \
        attention_mma_backward_key_kernel<HD, RECOMPUTE>                       \
            <<<grid, kThreads, key_bytes, stream>>>(                           \
                q, k, v, probabilities, lse, dout, row_dots, dk, dv, int(seq), \
                scale, add_k, add_v);                                          \
        launched = true;                                                       \
    }
#define CALL(HD)                                                               \
    if (recompute) { LAUNCH(HD, true) } else { LAUNCH(HD, false) }
    VITB200_MMA_DISPATCH(head_dim, CALL)
#undef CALL
#undef LAUNCH
    g_kernel_launches += launched ? 3 : 0;
    return launched;
}

}  // namespace vitb200
