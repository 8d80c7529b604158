// Whole-image 2-D transforms for DX = 256 on the 32-point register FFT (fft32.cuh): one CTA of 16
// warps per image, the 256 x 64 intermediate in shared memory, as in fft2d_trunc_kernel /
// ifft2d_pad_kernel of spectral_kernels.cuh -- but a signal is spread over R = len/32 ADJACENT lanes
// holding 32 samples each, so a thread needs ~100 registers and four warps share a scheduler
// instead of two (the 64-point image kernels run at 43 % issue utilisation with their latencies
// exposed), and a group's global accesses are contiguous (8 lanes x 8 bytes) without the
// pair-and-shuffle step.  No counterpart in the reference, which round-trips the X-transformed
// image through global memory (fusion_variants/2D_D_exp_fused_fft_cgemm_ifft/fused_trunc_2D.cu:188-192).
#pragma once
#include "fft32.cuh"
#include "spectral_kernels.cuh"

namespace tfno {

constexpr int kImage32Threads = 512;

// [rows][64] complex tile, 512-byte rows of 32 16-byte chunks; the low three bits of the chunk index
// are XOR-ed with the row and with the chunk's group of eight, so that (a) the eight lanes of a
// group storing chunks 4 apart, (b) column accesses of eight consecutive rows, both cover all banks.
TFNO_HD int swz32_chunk(int row, int c) { return (c & ~7) | ((c & 7) ^ ((row & 7) ^ ((c >> 3) & 3))); }
TFNO_HD int tile32_index(int row, int m) { return row * kModes + swz32_chunk(row, m >> 1) * 2 + (m & 1); }

inline size_t image32_smem_bytes(int DX, int DY) { return ((size_t)DX * kModes + (DX / 32) * 32 + (DY / 32) * 32) * sizeof(float2); }

// [image][DX][DY] -> [image][64][64]      RX = DX/32 (8), RY = DY/32 (4 or 8)
template <int RX, int RY>
__global__ void __launch_bounds__(kImage32Threads, 1) fft2d_trunc32_kernel(ImageParams p) {
    constexpr int DX = 32 * RX, DY = 32 * RY;
    static_assert(kImage32Threads == kModes * RX, "one X-pass round: 64 columns x RX lanes");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* sY = reinterpret_cast<float2*>(smem_raw);          // [DX][64] swizzled
    float2* twY = sY + DX * kModes;                             // [RY][32]
    float2* twX = twY + RY * 32;                                // [RX][32]
    const int tid = threadIdx.x;
    fill_forward_table32<RY>(twY, tid, kImage32Threads);
    fill_forward_table32<RX>(twX, tid, kImage32Threads, p.centered_x != 0);
    __syncthreads();
    for (long long img = blockIdx.x; img < p.nimg; img += gridDim.x) {
        const float2* src = p.in + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k;
        {
            constexpr int GROUPS = kImage32Threads / RY, PER = 64 / RY;
            const int g = tid / RY, r = tid % RY;
            const float2 coef = round1_coef32<RY>(r);
#pragma unroll 1
            for (int x0 = 0; x0 < DX; x0 += GROUPS) {
                const int x = x0 + g;
                const float2* row = src + (long long)x * DY + r;
                float2 v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __ldg(row + RY * i);
                // the rows of the next round (or of this CTA's next image) travel to the L2 meanwhile
                if (x0 + GROUPS < DX) prefetch_l2_block(src + (long long)(x0 + GROUPS) * DY, GROUPS * DY * 8, tid, kImage32Threads);
                else if (img + gridDim.x < p.nimg) {
                    const long long nx = img + gridDim.x;
                    prefetch_l2_block(p.in + (nx % p.per_k) * p.stride_b + (nx / p.per_k) * p.stride_k, GROUPS * DY * 8, tid, kImage32Threads);
                }
                forward_trunc32<RY>(v, twY, r, 1, coef);
#pragma unroll
                for (int j = 0; j < PER; j += 2) {
                    const int m = PER * r + j;
                    *reinterpret_cast<float4*>(sY + x * kModes + swz32_chunk(x, m >> 1) * 2) =
                        make_float4(v[slot32(j)].x, v[slot32(j)].y, v[slot32(j + 1)].x, v[slot32(j + 1)].y);
                }
            }
        }
        __syncthreads();
        {
            constexpr int PER = 64 / RX;
            const int ky = tid / RX, r = tid % RX;
            const float2 coef = round1_coef32<RX>(r);
            float2* dst = p.out + img * (long long)(kModes * kModes);
            float2 v[32];
#pragma unroll
            for (int n = 0; n < 32; ++n) v[n] = sY[tile32_index(RX * n + r, ky)];
            forward_trunc32<RX>(v, twX, r, 1, coef);
#pragma unroll
            for (int j = 0; j < PER; ++j) dst[(PER * r + j) * kModes + ky] = v[slot32(j)];
        }
        __syncthreads();
    }
}

// [image][64][64] -> zero-pad -> inverse along X into shared memory -> inverse along Y -> [image][DX][DY]
// INVERSE: true inverse (computed as swap(FFT(swap(u))), one copy of the 32-point code) or a second
// forward transform.
template <int RX, int RY, bool INVERSE>
__global__ void __launch_bounds__(kImage32Threads, 1) ifft2d_pad32_kernel(ImageParams p) {
    constexpr int DX = 32 * RX, DY = 32 * RY;
    static_assert(kImage32Threads == kModes * RX, "one X-pass round: 64 columns x RX lanes");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* sY = reinterpret_cast<float2*>(smem_raw);
    float2* twY = sY + DX * kModes;                             // [RY][32]
    float2* twX = twY + RY * 32;                                // [RX][32]
    const int tid = threadIdx.x;
    fill_inverse_table32_folded<RY>(twY, tid, kImage32Threads, make_float2(1.f, 0.f), INVERSE);
    fill_inverse_table32_folded<RX>(twX, tid, kImage32Threads, p.gain, INVERSE, INVERSE && p.centered_x != 0);
    __syncthreads();
    for (long long img = blockIdx.x; img < p.nimg; img += gridDim.x) {
        const float2* src = p.in + img * (long long)(kModes * kModes);
        float2* dst = p.out + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k;
        {
            const int ky = tid / RX, j1 = tid % RX;
            const float2 coef = inverse_fold_coef32<RX>(j1, INVERSE);
            float2 v[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) {
                const float2 lo = __ldg(src + m * kModes + ky), hi = __ldg(src + (m + 32) * kModes + ky);
                const float2 u = cmul(cmadd(lo, coef, hi), twX[tw_index<RX>(j1, m)]);
                v[m] = INVERSE ? make_float2(u.y, u.x) : u;
            }
            fft32<-1>(v);
#pragma unroll
            for (int j2 = 0; j2 < 32; ++j2) {
                const float2 o = v[slot32(j2)];
                sY[tile32_index(RX * j2 + j1, ky)] = INVERSE ? make_float2(o.y, o.x) : o;
            }
        }
        __syncthreads();
        {
            constexpr int GROUPS = kImage32Threads / RY;
            const int g = tid / RY, j1 = tid % RY;
            const float2 coef = inverse_fold_coef32<RY>(j1, INVERSE);
#pragma unroll 1
            for (int x0 = 0; x0 < DX; x0 += GROUPS) {
                const int x = x0 + g;
                float2 v[32];
                // u[m'] = T[m'] (C[m'] + c C[m'+32]); a 16-byte chunk holds modes 2c, 2c+1
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float4 lo = *reinterpret_cast<const float4*>(sY + x * kModes + swz32_chunk(x, c) * 2);
                    const float4 hi = *reinterpret_cast<const float4*>(sY + x * kModes + swz32_chunk(x, c + 16) * 2);
                    const float4 t = *reinterpret_cast<const float4*>(twY + tw_index<RY>(j1, 2 * c));
                    const float2 u0 = cmul(cmadd(make_float2(lo.x, lo.y), coef, make_float2(hi.x, hi.y)), make_float2(t.x, t.y));
                    const float2 u1 = cmul(cmadd(make_float2(lo.z, lo.w), coef, make_float2(hi.z, hi.w)), make_float2(t.z, t.w));
                    v[2 * c] = INVERSE ? make_float2(u0.y, u0.x) : u0;
                    v[2 * c + 1] = INVERSE ? make_float2(u1.y, u1.x) : u1;
                }
                fft32<-1>(v);
                // Lanes j1 and j1 ^ 1 own samples that alternate in memory: each stores 16 bytes (its own
                // sample and the neighbour's) for every second j2 and they swap the foreign halves with a
                // shuffle, so that a group writes a whole 128-byte line per instruction.
                const bool odd = (j1 & 1) != 0;
                float2* row = dst + (long long)x * DY + (odd ? RY : 0) + (j1 & ~1);
#pragma unroll
                for (int n2 = 0; n2 < 16; ++n2) {
                    const float2 a = v[slot32(2 * n2)], b = v[slot32(2 * n2 + 1)];
                    const float2 ev = INVERSE ? make_float2(a.y, a.x) : a;       // this lane's sample RY*(2*n2) + j1
                    const float2 od = INVERSE ? make_float2(b.y, b.x) : b;       // this lane's sample RY*(2*n2+1) + j1
                    const float2 send = odd ? ev : od;
                    float2 got;
                    got.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
                    got.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
                    *reinterpret_cast<float4*>(row + 2 * RY * n2) =
                        odd ? make_float4(got.x, got.y, od.x, od.y) : make_float4(ev.x, ev.y, got.x, got.y);
                }
            }
        }
        __syncthreads();
    }
}

}  // namespace tfno
