// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = act(A[M,K] . B[N,K]^T + bias + residual).
//
// Replaces the library GEMMs the original reaches through ONNX Runtime
// (reference src/apps/ort_app.h:511-516) with a hand-written sm_100a kernel:
//   * one elected thread issues TMA loads of 128 x 64 (A) and BN x 64 (B) bf16
//     tiles into 128-byte-swizzled shared memory, STAGES deep, tracked by
//     full/empty mbarriers;
//   * one elected thread issues tcgen05.mma (M=128, N=BN, K=16 per instruction)
//     with the fp32 accumulator in tensor memory, and releases each stage with
//     tcgen05.commit;
//   * four epilogue warps read the accumulator back with tcgen05.ld, apply bias,
//     residual and activation in registers and store bf16 (or fp32) rows.
// The A operand can instead be gathered row by row with cp.async (implicit-GEMM
// convolution: a row is the Cin-slice of one input pixel for one filter tap, zero
// for padding), which is how 3x3, 7x7 and strided 1x1 convolutions reuse this
// kernel.  All loads read this GPU's memory; no multicast is used.
// Every mbarrier wait is bounded; when one runs out the kernel records an error
// code in *status, stops issuing work, lets in-flight copies land, frees its
// tensor memory and returns.
#include "gemm_tcgen05.h"
#include "ptx.cuh"
#include "per_device.h"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;  // warp 0 producer, warp 1 mma, warps 2-5 epilogue
constexpr int CONV_THREADS = 320;  // warps 0-3 gather producers, warp 4 B-loader, warp 5 mma, warps 6-9 epilogue

__device__ __forceinline__ float gelu_f(float x) { return ptx::gelu_erf_fast(x); }

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

__device__ __forceinline__ void epilogue_store(const GemmEpilogue& ep, uint32_t tmem_base, int warp_q, int lane, int m0,
                                               int n0, int M, int N, int BN) {
  const int row = m0 + warp_q * 32 + lane;
  const bool vec_out = ((ep.ldo & 7) == 0) && (((uintptr_t)ep.out & 15) == 0);
  const bool vec_res = ((ep.ldr & 7) == 0) && (((uintptr_t)ep.residual & 15) == 0);
  for (int c = 0; c < BN; c += 32) {
    uint32_t r[32];
    ptx::tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp_q * 32) << 16) + (uint32_t)c, r);
    ptx::tmem_ld_wait();
    if (row >= M) continue;
    const int col0 = n0 + c;
    if (col0 >= N) continue;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
    if (ep.bias) {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col0 + j < N) v[j] += __ldg(ep.bias + col0 + j);
    }
    if (ep.residual) {
      const __nv_bfloat16* rp = ep.residual + (size_t)row * ep.ldr + col0;
      if (col0 + 32 <= N && vec_res) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 q = *reinterpret_cast<const uint4*>(rp + j);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
          for (int t = 0; t < 4; t++) {
            float2 f = __bfloat1622float2(h[t]);
            v[j + 2 * t] += f.x;
            v[j + 2 * t + 1] += f.y;
          }
        }
      } else {
        #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < N) v[j] += __bfloat162float(rp[j]);
      }
    }
    if (ep.act == GEMM_ACT_RELU) {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
    } else if (ep.act == GEMM_ACT_GELU) {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
    } else if (ep.act == GEMM_ACT_TANH) {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = tanhf(v[j]);
    }
    if (ep.out_fp32) {
      float* op = reinterpret_cast<float*>(ep.out) + (size_t)row * ep.ldo + col0;
      #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < N) op[j] = v[j];
    } else {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(ep.out) + (size_t)row * ep.ldo + col0;
      if (col0 + 32 <= N && vec_out) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 q;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
          for (int t = 0; t < 4; t++) h[t] = __floats2bfloat162_rn(v[j + 2 * t], v[j + 2 * t + 1]);
          *reinterpret_cast<uint4*>(op + j) = q;
        }
      } else {
        #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < N) op[j] = __float2bfloat16(v[j]);
      }
    }
  }
}

// ------------------------------------------------------------------ plain GEMM (A and B by TMA)
template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_bf16_tma(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, int M, int N, int K,
              GemmEpilogue ep, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = SmemLayout<BN>;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(&tmem_full_bar, 1);
    ptx::fence_mbar_init();
    s_error = 0;
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_smem, BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    if (ptx::elect_one()) {
      for (int kb = 0; kb < num_kb; kb++) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
          break;
        }
        ptx::mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
        uint8_t* sa = smem + (size_t)s * L::STAGE_BYTES;
        ptx::tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, m0);
        ptx::tma_load_2d(sa + L::A_BYTES, &tmap_b, &full_bar[s], kb * BK, n0);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb; kb++) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&full_bar[s], ph)) {
          atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t sa = ptx::smem_u32(smem + (size_t)s * L::STAGE_BYTES);
        const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++) {
          ptx::umma_bf16(tmem_base, ptx::umma_desc_sw128(sa + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2),
                         idesc, (kb | k) != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&empty_bar[s]);
      }
      (void)ok;
      ptx::umma_commit(&tmem_full_bar);  // arrives once every MMA issued so far has finished
    }
  } else {
    const int warp_q = warp & 3;  // TMEM lane quarter this warp may read
    if (ptx::mbar_wait(&tmem_full_bar, 0) && s_error == 0) {
      ptx::tc_fence_after();
      epilogue_store(ep, tmem_base, warp_q, lane, m0, n0, M, N, BN);
    } else if (lane == 0) {
      atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, s_error);
    __nanosleep(1000000);  // let copies that are still in flight land before the block leaves
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, BN);
  }
}

// ------------------------------------------------------------------ implicit-GEMM convolution (A gathered)
// Activations are NHWC bf16, filters [Cout][R][S][Cin] bf16 (K-major rows of
// length R*S*Cin).  GEMM view: M = N*OH*OW output pixels, N = Cout,
// K = R*S*Cin with Cin a multiple of 64, so one 64-wide K block is the
// Cin-slice [c0, c0+64) of one filter tap.
template <int BN, int STAGES>
__global__ void __launch_bounds__(CONV_THREADS)
conv_bf16_igemm(const __nv_bfloat16* __restrict__ in, const __grid_constant__ CUtensorMap tmap_w, ConvShape cs,
                GemmEpilogue ep, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = SmemLayout<BN>;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];   // 128 gather arrivals + 1 expect_tx arrival
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = cs.n * cs.oh * cs.ow, N = cs.cout;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int cblocks = cs.cin / BK;
  const int num_kb = cs.r * cs.s * cblocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 128 + 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(&tmem_full_bar, 1);
    ptx::fence_mbar_init();
    s_error = 0;
    ptx::prefetch_tmap(&tmap_w);
  }
  if (warp == 5) {
    ptx::tmem_alloc(&tmem_base_smem, BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp < 4) {
    // Gather producers: thread t owns row t of the A tile (one output pixel).
    const int r_row = threadIdx.x;
    const int m = m0 + r_row;
    const bool row_ok = m < M;
    int img = 0, oy = 0, ox = 0;
    if (row_ok) {
      img = m / (cs.oh * cs.ow);
      int rem = m - img * cs.oh * cs.ow;
      oy = rem / cs.ow;
      ox = rem - oy * cs.ow;
    }
    const int iy0 = oy * cs.stride - cs.pad, ix0 = ox * cs.stride - cs.pad;
    const uint32_t swz = (uint32_t)(r_row & 7);
    for (int kb = 0; kb < num_kb; kb++) {
      const int s = kb % STAGES;
      const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
      if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) {
        atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
        break;
      }
      const int tap = kb / cblocks, cb = kb - tap * cblocks;
      const int fr = tap / cs.s, fs = tap - fr * cs.s;
      const int iy = iy0 + fr, ix = ix0 + fs;
      const bool ok = row_ok && iy >= 0 && iy < cs.h && ix >= 0 && ix < cs.w;
      const __nv_bfloat16* src = ok ? in + (((size_t)img * cs.h + iy) * cs.w + ix) * cs.cin + cb * BK : in;
      uint8_t* dst_row = smem + (size_t)s * L::STAGE_BYTES + (size_t)r_row * 128;
#pragma unroll
      for (int c = 0; c < 8; c++) ptx::cp_async_16(dst_row + ((c ^ swz) << 4), src + c * 8, ok);
      ptx::cp_async_commit();
      // Keep one group in flight: publish the previous stage once its copies landed.
      if (kb > 0) {
        ptx::cp_async_wait<1>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(&full_bar[(kb - 1) % STAGES]);
      }
    }
    ptx::cp_async_wait<0>();
    ptx::fence_proxy_async_smem();
    if (num_kb > 0) ptx::mbar_arrive(&full_bar[(num_kb - 1) % STAGES]);
  } else if (warp == 4) {
    if (ptx::elect_one()) {
      for (int kb = 0; kb < num_kb; kb++) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
          break;
        }
        ptx::mbar_expect_tx(&full_bar[s], L::B_BYTES);
        ptx::tma_load_2d(smem + (size_t)s * L::STAGE_BYTES + L::A_BYTES, &tmap_w, &full_bar[s], kb * BK, n0);
      }
    }
  } else if (warp == 5) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
      for (int kb = 0; kb < num_kb; kb++) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        if (!ptx::mbar_wait(&full_bar[s], ph)) {
          atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t sa = ptx::smem_u32(smem + (size_t)s * L::STAGE_BYTES);
        const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++) {
          ptx::umma_bf16(tmem_base, ptx::umma_desc_sw128(sa + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2),
                         idesc, (kb | k) != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&empty_bar[s]);
      }
      ptx::umma_commit(&tmem_full_bar);
    }
  } else {
    const int warp_q = warp & 3;
    if (ptx::mbar_wait(&tmem_full_bar, 0) && s_error == 0) {
      ptx::tc_fence_after();
      epilogue_store(ep, tmem_base, warp_q, lane, m0, n0, M, N, BN);
    } else if (lane == 0) {
      atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, s_error);
    __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == 5) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, BN);
  }
}

cudaError_t encode_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->TensorMapEncodeTiled) return cudaErrorNotSupported;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d->TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <typename F>
cudaError_t set_smem(F f, int bytes) {
  return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int BN, int STAGES>
cudaError_t launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, int M, int N, int K, const GemmEpilogue& ep,
                        uint32_t* status, cudaStream_t st) {
  static PerDeviceFlag attr;
  const int dev = PerDeviceFlag::current();
  const int smem = STAGES * SmemLayout<BN>::STAGE_BYTES + 1024;
  if (attr.needed(dev)) {
    cudaError_t e = set_smem(gemm_bf16_tma<BN, STAGES>, smem);
    if (e != cudaSuccess) return e;
    attr.set(dev);
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_bf16_tma<BN, STAGES><<<grid, GEMM_THREADS, smem, st>>>(ta, tb, M, N, K, ep, status);
  return cudaGetLastError();
}

template <int BN, int STAGES>
cudaError_t launch_conv(const __nv_bfloat16* in, const CUtensorMap& tw, const ConvShape& cs, const GemmEpilogue& ep,
                        uint32_t* status, cudaStream_t st) {
  static PerDeviceFlag attr;
  const int dev = PerDeviceFlag::current();
  const int smem = STAGES * SmemLayout<BN>::STAGE_BYTES + 1024;
  if (attr.needed(dev)) {
    cudaError_t e = set_smem(conv_bf16_igemm<BN, STAGES>, smem);
    if (e != cudaSuccess) return e;
    attr.set(dev);
  }
  const int M = cs.n * cs.oh * cs.ow;
  dim3 grid((cs.cout + BN - 1) / BN, (M + BM - 1) / BM);
  conv_bf16_igemm<BN, STAGES><<<grid, CONV_THREADS, smem, st>>>(in, tw, cs, ep, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t srpc_gemm_bf16(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                           uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if ((lda % 8) || (ldb % 8) || (K % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return cudaErrorInvalidValue;
  const int bn = (N <= 64) ? 64 : 128;
  CUtensorMap ta, tb;
  cudaError_t e = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (e != cudaSuccess) return e;
  e = encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, (uint32_t)bn);
  if (e != cudaSuccess) return e;
  if (bn == 64) return launch_gemm<64, 4>(ta, tb, M, N, K, ep, status, stream);
  return launch_gemm<128, 3>(ta, tb, M, N, K, ep, status, stream);
}

cudaError_t srpc_conv_bf16(const void* in, const void* weight, const ConvShape& cs, const GemmEpilogue& ep,
                           uint32_t* status, cudaStream_t stream) {
  if (cs.cin % BK || cs.cout % 8) return cudaErrorInvalidValue;
  if (((uintptr_t)in & 15) || ((uintptr_t)weight & 15)) return cudaErrorInvalidValue;
  const int K = cs.r * cs.s * cs.cin;
  const int bn = (cs.cout <= 64) ? 64 : 128;
  CUtensorMap tw;
  cudaError_t e = encode_2d(&tw, weight, (uint64_t)K, (uint64_t)cs.cout, (uint64_t)K * 2, BK, (uint32_t)bn);
  if (e != cudaSuccess) return e;
  if (bn == 64) return launch_conv<64, 4>((const __nv_bfloat16*)in, tw, cs, ep, status, stream);
  return launch_conv<128, 3>((const __nv_bfloat16*)in, tw, cs, ep, status, stream);
}
