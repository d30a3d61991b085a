// The decayed outer-product recurrence of seqmix.cu for prompt portions, in its chunk-parallel form on the tensor cores.
//
//   S_t = a_t S_(t-1) + (c_t k_t) v_t^T,   y_t = S_t^T q_t + d v_t          (S: D x V per head, fp32)
//
// Over a chunk of C = 64 consecutive tokens with L_t = sum_{u <= t} log a_u (inside the chunk) and S_in the state before
// its first token:
//
//   y_t   = e^{L_t} S_in^T q_t  +  sum_{j <= t} e^{L_t - L_j} c_j (q_t . k_j) v_j
//   S_out = e^{L_last} S_in     +  sum_j e^{L_last - L_j} c_j k_j v_j^T
//
// so the work of a chunk is four small matrix products (Q K^T, P V, Q S_in, K^T V~) on mma.sync m16n8k16 with bf16
// operands and fp32 accumulation. What stays fp32: the state (it lives in accumulator registers for the whole portion
// and is read out as a bf16 high part plus a bf16 remainder, two MMAs, so the read-out keeps ~16 bits), the logarithms,
// their running sums and every exponential, the step sizes c_t; the decay weights multiply fp32 accumulators or fp32
// inputs before the one rounding to bf16 that any tensor-core operand gets. Every exponent is a difference L_t - L_j
// with j <= t, hence <= 0: nothing overflows however strong the decay. log a_t is clamped at -80 (a_t = 0 would make
// the differences undefined; e^-80 of a state is below fp32 resolution of anything added to it).
//
// One CTA = one sequence x one head x 64 value columns, eight warps: a PAIR of warps owns 16 value columns. The state
// tile is kept TRANSPOSED (rows = value columns, columns = key dimensions) so that the accumulator fragments of S^T
// turn into A fragments of S^T Q^T in registers, as a softmax kernel turns its probabilities into the A operand of P V.
// Inside a pair, each warp holds one half of the key dimensions of the state and produces one half of the chunk's token
// columns of the output: both compute their half of the sum over key dimensions for all 64 tokens and hand the partner
// the 32 columns it owns through shared memory. Halving the per-warp tiles is what lets sixteen warps live on an SM;
// with four warps of 246 registers the kernel ran at one warp per scheduler and waited on instruction latency.
// Sequences are walked as in seqmix.cu: rows [seq_start, seq_start + seq_count), state slot seq_slot, zero state when
// seq_pos0 == 0.
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

constexpr int kScC = 64;   // tokens per chunk
constexpr int kScV = 64;   // value columns per CTA
constexpr int kScT = 256;  // threads per CTA

__device__ __forceinline__ float silu_sc(float x) { return x / (1.f + expf(-x)); }

template <int D>
__global__ void __launch_bounds__(kScT, 2)
scan_chunked_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                    const float* __restrict__ v, long long ldv, int H, int G, int V,
                    const float* __restrict__ decay_head, const float* __restrict__ decay_tok,
                    const float* __restrict__ kscale_tok, const float* __restrict__ skip, int act,
                    float* __restrict__ state, float* __restrict__ y, long long ldy,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                    const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int vec) {
    constexpr int LQ = D + 8, LV = kScV + 8, LP = kScC + 8;   // padded rows: ldmatrix without bank conflicts
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [C][D]
    __nv_bfloat16* sK = sQ + kScC * LQ;                               // [C][D]
    __nv_bfloat16* sV = sK + kScC * LQ;                               // [C][64]  v_j
    __nv_bfloat16* sW = sV + kScC * LV;                               // [C][64]  e^{L_last - L_j} c_j v_j
    __nv_bfloat16* sP = sW + kScC * LV;                               // [C][C]   e^{L_t - L_j} c_j (q_t . k_j), j <= t
    float* sL = reinterpret_cast<float*>(sP + kScC * LP);             // [C] running sums of log a, per half of the chunk
    float* sC = sL + kScC;                                            // [C] c_j (0 for rows past the portion)
    float* sX = sC + kScC;                                            // [8 warps][16][32] partial sums for the partner
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kScV;
    const int n = seq_count[s];
    if (n <= 0) return;
    const long long r0 = seq_start[s];
    const int g = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = warp & 1;                   // which half of the key dimensions / of the token columns
    const int vw = (warp >> 1) * 16;
    constexpr int DH = D / 2;                    // key dimensions of the state per warp
    const int vr = v0 + vw + (lane >> 2);        // value column of accumulator elements 0, 1 (elements 2, 3: + 8)
    const int c2 = 2 * (lane & 3);               // first of this thread's two columns inside an 8-wide tile

    float S[DH / 8][4];
    float* st = state + (static_cast<long long>(seq_slot[s]) * H + h) * D * V;
    const bool fresh = seq_pos0[s] == 0;
#pragma unroll
    for (int nd = 0; nd < DH / 8; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int vv = vr + 8 * (e >> 1), d = half * DH + nd * 8 + c2 + (e & 1);
            S[nd][e] = (!fresh && vv < V) ? st[static_cast<long long>(d) * V + vv] : 0.f;
        }
    const float la_head = decay_head ? fmaxf(logf(decay_head[h]), -80.f) : 0.f;
    const float dskip = skip ? skip[h] : 0.f;
    auto Lc = [&](int t) { return sL[t] + (t >= 32 ? sL[31] : 0.f); };

    // Decay and step size of this thread's token (threads 0 .. 63) are fetched one chunk ahead into registers, and the
    // rows of the next chunk are pulled into L2 while this chunk's products run, so that what a chunk waits for is one
    // L2 round trip instead of several trips to HBM.
    float a_next = 1.f, c_next = 0.f;
    auto fetch_decay = [&](int c0n) {
        a_next = 1.f, c_next = 0.f;   // rows past the portion: no decay, no contribution
        if (threadIdx.x < kScC && c0n + static_cast<int>(threadIdx.x) < n) {
            const long long row = r0 + c0n + threadIdx.x;
            if (decay_tok) a_next = decay_tok[row * H + h];
            c_next = kscale_tok ? kscale_tok[row * H + h] : 1.f;
        }
    };
    auto pull_l2 = [&](int c0n) {
        const int cnn = min(kScC, n - c0n);
        constexpr int LQK = (D * 4 + 127) / 128 + 1, LVV = (kScV * 4 + 127) / 128 + 1;   // 128-byte lines a row may touch
        for (int e = threadIdx.x; e < cnn * LQK; e += kScT) {
            const int i = e / LQK, l = e - i * LQK;
            const long long row = r0 + c0n + i;
            if (l * 32 < D + 31) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(q + row * ldq + g * D + min(l * 32, D - 1)));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(k + row * ldk + g * D + min(l * 32, D - 1)));
            }
        }
        const int nv = min(kScV, V - v0);
        for (int e = threadIdx.x; e < cnn * LVV; e += kScT) {
            const int i = e / LVV, l = e - i * LVV;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(v + (r0 + c0n + i) * ldv + static_cast<long long>(h) * V + v0 +
                                                          min(l * 32, nv - 1)));
        }
    };
    fetch_decay(0);

    for (int c0 = 0; c0 < n; c0 += kScC) {
        const int cn = min(kScC, n - c0);
        __syncthreads();   // the previous chunk's tiles have been consumed
        if (threadIdx.x < kScC) {
            const int t = threadIdx.x;
            float la = 0.f;
            const float c = c_next;
            if (t < cn) la = decay_tok ? fmaxf(logf(a_next), -80.f) : la_head;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float x = __shfl_up_sync(0xffffffffu, la, o);
                if (lane >= o) la += x;
            }
            sL[t] = la;
            sC[t] = c;
        }
        __syncthreads();
        const float Llast = Lc(kScC - 1);
        // Tiles: loads are issued in batches ahead of their use (a chunk is short, so memory latency is what a naive
        // element loop would spend its time on); 16-byte loads when pointers, pitches and sizes allow.
        if (vec & 1) {
            constexpr int IT = kScC * D / 4 / kScT, U = IT;   // at most 8: one batch
#pragma unroll 1
            for (int it = 0; it < IT; it += U) {
                float4 xq[U], xk[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / (D / 4), d = (e - i * (D / 4)) * 4;
                    xq[u] = xk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (i < cn) {
                        xq[u] = *reinterpret_cast<const float4*>(q + (r0 + c0 + i) * ldq + g * D + d);
                        xk[u] = *reinterpret_cast<const float4*>(k + (r0 + c0 + i) * ldk + g * D + d);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / (D / 4), d = (e - i * (D / 4)) * 4;
                    if (act) {
                        xq[u] = make_float4(silu_sc(xq[u].x), silu_sc(xq[u].y), silu_sc(xq[u].z), silu_sc(xq[u].w));
                        xk[u] = make_float4(silu_sc(xk[u].x), silu_sc(xk[u].y), silu_sc(xk[u].z), silu_sc(xk[u].w));
                    }
                    *reinterpret_cast<uint2*>(sQ + i * LQ + d) = make_uint2(pack_bf16(xq[u].x, xq[u].y), pack_bf16(xq[u].z, xq[u].w));
                    *reinterpret_cast<uint2*>(sK + i * LQ + d) = make_uint2(pack_bf16(xk[u].x, xk[u].y), pack_bf16(xk[u].z, xk[u].w));
                }
            }
        } else {
            constexpr int IT = kScC * D / kScT, U = (IT % 16 == 0) ? 16 : 8;
#pragma unroll 1
            for (int it = 0; it < IT; it += U) {
                float xq[U], xk[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / D, d = e - i * D;
                    xq[u] = xk[u] = 0.f;
                    if (i < cn) {
                        xq[u] = q[(r0 + c0 + i) * ldq + g * D + d];
                        xk[u] = k[(r0 + c0 + i) * ldk + g * D + d];
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / D, d = e - i * D;
                    if (act) {
                        xq[u] = silu_sc(xq[u]);
                        xk[u] = silu_sc(xk[u]);
                    }
                    sQ[i * LQ + d] = __float2bfloat16_rn(xq[u]);
                    sK[i * LQ + d] = __float2bfloat16_rn(xk[u]);
                }
            }
        }
        if (vec & 2) {
            constexpr int IT = kScC * kScV / 4 / kScT, U = 4;
#pragma unroll 1
            for (int it = 0; it < IT; it += U) {
                float4 xv[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / (kScV / 4), j = (e - i * (kScV / 4)) * 4;
                    xv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (i < cn && v0 + j < V)
                        xv[u] = *reinterpret_cast<const float4*>(v + (r0 + c0 + i) * ldv + static_cast<long long>(h) * V + v0 + j);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / (kScV / 4), j = (e - i * (kScV / 4)) * 4;
                    if (act) xv[u] = make_float4(silu_sc(xv[u].x), silu_sc(xv[u].y), silu_sc(xv[u].z), silu_sc(xv[u].w));
                    const float w = expf(Llast - Lc(i)) * sC[i];
                    *reinterpret_cast<uint2*>(sV + i * LV + j) = make_uint2(pack_bf16(xv[u].x, xv[u].y), pack_bf16(xv[u].z, xv[u].w));
                    *reinterpret_cast<uint2*>(sW + i * LV + j) =
                        make_uint2(pack_bf16(xv[u].x * w, xv[u].y * w), pack_bf16(xv[u].z * w, xv[u].w * w));
                }
            }
        } else {
            constexpr int IT = kScC * kScV / kScT, U = 8;
#pragma unroll 1
            for (int it = 0; it < IT; it += U) {
                float xv[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / kScV, j = e - i * kScV;
                    xv[u] = 0.f;
                    if (i < cn && v0 + j < V) xv[u] = v[(r0 + c0 + i) * ldv + static_cast<long long>(h) * V + v0 + j];
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = threadIdx.x + (it + u) * kScT, i = e / kScV, j = e - i * kScV;
                    if (act) xv[u] = silu_sc(xv[u]);
                    sV[i * LV + j] = __float2bfloat16_rn(xv[u]);
                    sW[i * LV + j] = __float2bfloat16_rn(xv[u] * (expf(Llast - Lc(i)) * sC[i]));
                }
            }
        }
        __syncthreads();

        // ---- what the state before the chunk contributes: Y^T = S_in^T Q^T, column t scaled by e^{L_t} ------------
        float acc[4][4];   // Y^T: this pair's 16 value columns x this warp's 32 token columns
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        if (c0 + kScC < n) {
            fetch_decay(c0 + kScC);
            pull_l2(c0 + kScC);
        }
        const bool carry = !(fresh && c0 == 0);   // a state to read out (none before a sequence's first chunk)
        if (carry) {
            float part[kScC / 8][4];
#pragma unroll
            for (int i = 0; i < kScC / 8; ++i) part[i][0] = part[i][1] = part[i][2] = part[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < DH / 16; ++kk) {
                uint32_t ah[4], al[4];
#pragma unroll
                for (int f = 0; f < 4; ++f) {
                    const float x0 = S[2 * kk + (f >> 1)][2 * (f & 1)], x1 = S[2 * kk + (f >> 1)][2 * (f & 1) + 1];
                    ah[f] = pack_bf16(x0, x1);
                    al[f] = pack_bf16(x0 - bf16lo(ah[f]), x1 - bf16hi(ah[f]));
                }
#pragma unroll
                for (int nb2 = 0; nb2 < kScC / 16; ++nb2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(smem_u32(sQ + (nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * LQ + half * DH + kk * 16 +
                                     ((lane >> 3) & 1) * 8),
                            b0, b1, b2, b3);
                    mma_bf16(part[2 * nb2], ah, b0, b1);
                    mma_bf16(part[2 * nb2 + 1], ah, b2, b3);
                    mma_bf16(part[2 * nb2], al, b0, b1);
                    mma_bf16(part[2 * nb2 + 1], al, b2, b3);
                }
            }
            // keep the token tiles this warp owns, hand the other four to the partner
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sX[(warp * 16 + i * 4 + e) * 32 + lane] = half ? part[i][e] : part[4 + i][e];
                    acc[i][e] = half ? part[4 + i][e] : part[i][e];
                }
        }

        // ---- P: 16 rows x 32 keys of (Q K^T) per warp, with the decay between key and query; keys after the query 0 ---
        {
            const int rt = warp >> 1;   // row tile of this warp; its key columns are [32 half, 32 half + 32)
            float sc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t qf[4];
                ldsm_x4(smem_u32(sQ + (rt * 16 + (lane & 15)) * LQ + ks * 16 + (lane >> 4) * 8), qf[0], qf[1], qf[2], qf[3]);
#pragma unroll
                for (int n2 = 0; n2 < 2; ++n2) {
                    const int nb2 = 2 * half + n2;
                    if (nb2 > rt) continue;   // every key of the tile lies after this warp's rows (warp-uniform)
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(smem_u32(sK + (nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * LQ + ks * 16 + ((lane >> 3) & 1) * 8),
                            b0, b1, b2, b3);
                    mma_bf16(sc[2 * n2], qf, b0, b1);
                    mma_bf16(sc[2 * n2 + 1], qf, b2, b3);
                }
            }
            const int t0 = rt * 16 + (lane >> 2);
            const float Lt0 = Lc(t0), Lt1 = Lc(t0 + 8);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = t0 + 8 * (e >> 1), j = (4 * half + i) * 8 + c2 + (e & 1);
                    p[e] = (j <= t) ? sc[i][e] * (expf(((e >> 1) ? Lt1 : Lt0) - Lc(j)) * sC[j]) : 0.f;
                }
                *reinterpret_cast<uint32_t*>(sP + t0 * LP + (4 * half + i) * 8 + c2) = pack_bf16(p[0], p[1]);
                *reinterpret_cast<uint32_t*>(sP + (t0 + 8) * LP + (4 * half + i) * 8 + c2) = pack_bf16(p[2], p[3]);
            }
        }
        __syncthreads();   // P complete; the partner's partial sums are in place

        // ---- the state's share of this warp's 32 token columns: both halves of the key dimensions, column t x e^{L_t} --
        if (carry) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = (4 * half + i) * 8 + c2;
                const float e0 = expf(Lc(t)), e1 = expf(Lc(t + 1));
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    acc[i][e] = (acc[i][e] + sX[((warp ^ 1) * 16 + i * 4 + e) * 32 + lane]) * ((e & 1) ? e1 : e0);
            }
        }

        // ---- inside the chunk: Y^T += V^T P^T -------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < kScC / 16; ++kk) {
            uint32_t a[4];
            ldsm_x4_t(smem_u32(sV + (kk * 16 + (lane >> 4) * 8 + (lane & 7)) * LV + vw + ((lane >> 3) & 1) * 8), a[0], a[1],
                      a[2], a[3]);
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {
                const int nb2 = 2 * half + n2;
                if (kk > nb2) continue;   // keys after every query of the tile
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(sP + (nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * LP + kk * 16 + ((lane >> 3) & 1) * 8), b0,
                        b1, b2, b3);
                mma_bf16(acc[2 * n2], a, b0, b1);
                mma_bf16(acc[2 * n2 + 1], a, b2, b3);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i += 2) {
            float xs[8];
#pragma unroll
            for (int f = 0; f < 8; ++f) {
                const int t = (4 * half + i + (f >> 2)) * 8 + c2 + (f & 1), vv = vr + 8 * ((f >> 1) & 1);
                xs[f] = (skip && t < cn && vv < V) ? v[(r0 + c0 + t) * ldv + static_cast<long long>(h) * V + vv] : 0.f;
            }
#pragma unroll
            for (int f = 0; f < 8; ++f) {
                const int t = (4 * half + i + (f >> 2)) * 8 + c2 + (f & 1), vv = vr + 8 * ((f >> 1) & 1);
                if (t >= cn || vv >= V) continue;
                float out = acc[i + (f >> 2)][f & 3];
                if (skip) out = fmaf(dskip, act ? silu_sc(xs[f]) : xs[f], out);
                y[(r0 + c0 + t) * ldy + static_cast<long long>(h) * V + vv] = out;
            }
        }

        // ---- the state after the chunk: S^T = e^{L_last} S^T + V~^T K ------------------------------------------------
        const float dl = expf(Llast);
#pragma unroll
        for (int nd = 0; nd < DH / 8; ++nd) {
            S[nd][0] *= dl;
            S[nd][1] *= dl;
            S[nd][2] *= dl;
            S[nd][3] *= dl;
        }
#pragma unroll
        for (int kk = 0; kk < kScC / 16; ++kk) {
            if (kk * 16 >= cn) continue;   // rows past the portion are zero
            uint32_t a[4];
            ldsm_x4_t(smem_u32(sW + (kk * 16 + (lane >> 4) * 8 + (lane & 7)) * LV + vw + ((lane >> 3) & 1) * 8), a[0], a[1],
                      a[2], a[3]);
#pragma unroll
            for (int nb2 = 0; nb2 < DH / 16; ++nb2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(smem_u32(sK + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LQ + half * DH + nb2 * 16 +
                                   (lane >> 4) * 8),
                          b0, b1, b2, b3);
                mma_bf16(S[2 * nb2], a, b0, b1);
                mma_bf16(S[2 * nb2 + 1], a, b2, b3);
            }
        }
    }
#pragma unroll
    for (int nd = 0; nd < DH / 8; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int vv = vr + 8 * (e >> 1), d = half * DH + nd * 8 + c2 + (e & 1);
            if (vv < V) st[static_cast<long long>(d) * V + vv] = S[nd][e];
        }
}

template <int D>
static int launch_scan_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                               int H, int G, int V, const float* decay_head, const float* decay_tok,
                               const float* kscale_tok, const float* skip, int act, float* state, float* y,
                               long long ldy, const int* seq_start, const int* seq_count, const int* seq_pos0,
                               const int* seq_slot, int n_seqs, int flags, cudaStream_t stream) {
    const int smem = 2 * kScC * (D + 8) * 2 + 2 * kScC * (kScV + 8) * 2 + kScC * (kScC + 8) * 2 + 2 * kScC * 4 +
                     8 * 16 * 32 * 4;
    static bool attr_done = false;
    if (!attr_done) {
        ATX_CUDA(cudaFuncSetAttribute(scan_chunked_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(n_seqs, H, (V + kScV - 1) / kScV);
    cfg.blockDim = dim3(kScT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    // bit 0: q / k rows can be read 16 bytes at a time; bit 1: v rows
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const int vec = ((al16(q) && al16(k) && ldq % 4 == 0 && ldk % 4 == 0) ? 1 : 0) |
                    ((al16(v) && ldv % 4 == 0 && V % 4 == 0) ? 2 : 0);
    ATX_CUDA(cudaLaunchKernelEx(&cfg, scan_chunked_kernel<D>, q, ldq, k, ldk, v, ldv, H, G, V, decay_head, decay_tok,
                                kscale_tok, skip, act, state, y, ldy, seq_start, seq_count, seq_pos0, seq_slot, vec));
    return ATX_OK;
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_linear_recurrence_chunked_supported(int D) {
    return (D == 32 || D == 64 || D == 96 || D == 128) ? 1 : 0;
}

int atx_linear_recurrence_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v,
                                  long long ldv, int H, int G, int D, int V, const float* decay_head,
                                  const float* decay_tok, const float* kscale_tok, const float* skip, int act,
                                  float* state, float* y, long long ldy, const int* seq_start, const int* seq_count,
                                  const int* seq_pos0, const int* seq_slot, int n_seqs, int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k && v && state && y && seq_start && seq_count && seq_pos0 && seq_slot,
                "atx_linear_recurrence_chunked: null pointer");
    ATX_REQUIRE((decay_head != nullptr) != (decay_tok != nullptr),
                "atx_linear_recurrence_chunked: exactly one of decay_head / decay_tok");
    ATX_REQUIRE(n_seqs > 0 && H > 0 && G > 0 && H % G == 0 && V > 0 && atx_linear_recurrence_chunked_supported(D),
                "atx_linear_recurrence_chunked: bad shape n_seqs=%d H=%d G=%d D=%d V=%d", n_seqs, H, G, D, V);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
#define ATX_SCAN_CASE(D_)                                                                                                \
    case D_:                                                                                                             \
        return launch_scan_chunked<D_>(q, ldq, k, ldk, v, ldv, H, G, V, decay_head, decay_tok, kscale_tok, skip, act,   \
                                       state, y, ldy, seq_start, seq_count, seq_pos0, seq_slot, n_seqs, flags, cs)
    switch (D) {
        ATX_SCAN_CASE(32);
        ATX_SCAN_CASE(64);
        ATX_SCAN_CASE(96);
        ATX_SCAN_CASE(128);
    }
#undef ATX_SCAN_CASE
    return ATX_OK;
}

}  // extern "C"
