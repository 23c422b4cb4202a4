// Blackwell (sm_100a) primitives as inline PTX: mbarriers with BOUNDED waits, TMA tensor copies
// (cp.async.bulk.tensor, never with cluster multicast), tcgen05 tensor-memory allocation, MMA issue,
// commit and loads, shared-memory matrix descriptors for 128-byte swizzled tiles, and the host-side
// tensor-map encoder (cuTensorMapEncodeTiled resolved through the runtime, so the library does not
// link against libcuda).
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

// ------------------------------------------------------------------------------------------------ host: tensor maps
typedef CUresult (*NnbEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline NnbEncodeTiled nnb_encode_fn() {
  // The encoder is a driver call and needs a current context. A thread that has only ever been handed work (an autograd
  // worker whose device is already "current" for PyTorch) may not have bound the primary context yet: bind it once per thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  static NnbEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<NnbEncodeTiled>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] with `row_stride_bytes`; box = [box_rows, box_cols]; 128-byte
// swizzle (box_cols * elem_bytes must be 128). Returns false on failure (message set).
static inline bool nnb_make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                                    uint64_t rows, uint64_t cols, uint64_t row_stride_bytes, uint32_t box_rows,
                                    uint32_t box_cols, const char* what) {
  NnbEncodeTiled enc = nnb_encode_fn();
  if (!enc) { nnb_set_error("%s: cuTensorMapEncodeTiled is not available", what); return false; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) {
    nnb_set_error("%s: TMA needs a 16-byte aligned base and row stride (base=%p stride=%llu)", what, base,
                  (unsigned long long)row_stride_bytes);
    return false;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = (box_cols * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (box_cols * elem_bytes == 64) ? CU_TENSOR_MAP_SWIZZLE_64B
                          : (box_cols * elem_bytes == 32) ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    nnb_set_error("%s: cuTensorMapEncodeTiled failed with %d (rows=%llu cols=%llu stride=%llu box=%ux%u)", what, (int)r,
                  (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_stride_bytes, box_rows, box_cols);
    return false;
  }
  return true;
}

// 3-D variant: dims (inner=cols, mid=rows, outer=batch) with two byte strides.
static inline bool nnb_make_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                                    uint64_t d2, uint64_t d1, uint64_t d0, uint64_t stride1_bytes, uint64_t stride2_bytes,
                                    uint32_t box1, uint32_t box0, const char* what) {
  NnbEncodeTiled enc = nnb_encode_fn();
  if (!enc) { nnb_set_error("%s: cuTensorMapEncodeTiled is not available", what); return false; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) {
    nnb_set_error("%s: TMA needs 16-byte aligned base and strides", what);
    return false;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = (box0 * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { nnb_set_error("%s: cuTensorMapEncodeTiled(3d) failed with %d", what, (int)r); return false; }
  return true;
}

// 4-D variant for attention operands: dims (d0 = head_dim [contiguous], d1 = heads, d2 = t, d3 = batch)
// with byte strides for d1..d3; box = (box0, 1, box2, 1); 128-byte swizzle when box0 * elem_bytes == 128.
static inline bool nnb_make_tmap_4d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
                                    uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1_bytes,
                                    uint64_t s2_bytes, uint64_t s3_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                                    const char* what) {
  NnbEncodeTiled enc = nnb_encode_fn();
  if (!enc) { nnb_set_error("%s: cuTensorMapEncodeTiled is not available", what); return false; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15) || (s3_bytes & 15)) {
    nnb_set_error("%s: TMA needs a 16-byte aligned base and strides (base=%p strides=%llu,%llu,%llu)", what, base,
                  (unsigned long long)s1_bytes, (unsigned long long)s2_bytes, (unsigned long long)s3_bytes);
    return false;
  }
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1_bytes, s2_bytes, s3_bytes};
  cuuint32_t box[4] = {box0, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapSwizzle sw = (box0 * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    nnb_set_error("%s: cuTensorMapEncodeTiled(4d) failed with %d (dims %llu,%llu,%llu,%llu)", what, (int)r,
                  (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, (unsigned long long)d3);
    return false;
  }
  return true;
}

// Optional phase timers (clock64) of one thread of CTA (0,0,0); compiled in only with -DNNB_PROFILE.
#ifdef NNB_PROFILE
static __device__ unsigned long long g_flash_prof[8];
#define NNB_PROF_DECL long long prof_t = 0; unsigned long long prof_acc[5] = {0, 0, 0, 0, 0}
#define NNB_PROF_T0 prof_t = clock64()
#define NNB_PROF_ADD(i) do { const long long now_ = clock64(); prof_acc[i] += now_ - prof_t; prof_t = now_; } while (0)
#define NNB_PROF_FLUSH_N(n_) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64) { \
  for (int i_ = 0; i_ < 5; ++i_) g_flash_prof[i_] = prof_acc[i_]; g_flash_prof[5] = (n_); } } while (0)
#define NNB_PROF_FLUSH NNB_PROF_FLUSH_N(n_kv)
#else
#define NNB_PROF_DECL
#define NNB_PROF_T0
#define NNB_PROF_ADD(i)
#define NNB_PROF_FLUSH
#define NNB_PROF_FLUSH_N(n_)
#endif

#ifdef __CUDACC__
namespace sm100 {

constexpr uint32_t kSpinLimit = 1u << 24;  // bounded waits: ~seconds, then the kernel gives up cleanly

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile("{\n.reg .b32 r;\n.reg .pred p;\nelect.sync r|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait. Returns false (and raises *abort_flag, a shared-memory word every role polls) when
// the phase did not complete within kSpinLimit polls or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// ---- TMA (tensor maps live in kernel parameters: __grid_constant__ const CUtensorMap)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// Bring one tile of a tensor map into L2 only (no shared-memory destination, nothing to wait for): a later tma_load_2d of the
// same box then pays L2 latency instead of HBM latency.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_group() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// ---- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], 16-bit inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// A operand from tensor memory (e.g. softmax probabilities written back with tcgen05.st).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Block-scaled 8-bit MMA (MXFP8): D[tmem] (+)= (A * sfa) (B * sfb)^T with one e8m0 scale per 32 contraction elements of every
// row; K = 32 per instruction. The scales sit in tensor memory (32-bit column c, lane l holds the 4 scale bytes of row
// 32 c' + l of 4 consecutive K blocks, replicated over the four lane quarters); the byte used is picked by the scale ids in
// the instruction descriptor AND by bits 30-31 of the scale addresses.
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                          uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// Shared memory -> tensor memory copy of 32 rows x 16 bytes, broadcast to the four lane quarters: the scale factors of 128
// rows x 4 K-blocks (row r at byte (r % 32) * 16 + (r / 32) * 4 of the 512-byte chunk) land in 4 columns.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// Descriptor of an unswizzled K-major block whose 8-row groups of 16-byte rows are `sbo_bytes` apart (128 when contiguous).
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100; layout type 0 = no swizzle
  return d;
}
// Instruction descriptor for kind::mxf8f6f4.block_scale with e4m3 operands (format 0), K-major, e8m0 scales (bit 23);
// the scale ids (bits 4-5 for B, 29-30 for A) are OR-ed in per instruction.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int M, int N) {
  return ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24);
}
// Plain bulk copy global -> shared with mbarrier completion (16-byte aligned addresses and size).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread t reads lane t of the
// warp's lane quarter).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

// ---- descriptors
// Shared-memory matrix descriptor for a 128-byte swizzled tile (base 1024-byte aligned).
//   K-major  : rows of 64 16-bit elements (128 B); SBO = 1024 (next 8 rows); LBO unused.
//   MN-major : k-rows of 64 MN-elements (128 B); SBO = 1024 (next 8 k-rows); LBO = bytes between
//              consecutive 64-element MN groups (one TMA box).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A/B format (0 = f16, 1 = bf16), majors
// (0 = K-major, 1 = MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_f16(int fmt_ab, int a_mn, int b_mn, int M, int N) {
  return (1u << 4) | ((uint32_t)fmt_ab << 7) | ((uint32_t)fmt_ab << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Two fp32 values rounded to the 16-bit operand format of the kernel (F16: IEEE half, otherwise bfloat16), packed low | high.
template <bool F16>
__device__ __forceinline__ uint32_t pack2_16(float a, float b) {
  if constexpr (F16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <bool F16> struct Operand16 { using type = __nv_bfloat16; };
template <> struct Operand16<true> { using type = __half; };

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Barrier among `nthreads` threads that also ORs a flag: every participant gets the same answer, so
// a role whose bounded wait ran out can make all its threads leave together instead of stranding
// the others at the next barrier.
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool flag) {
  uint32_t out;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 p, %3, 0;\nbarrier.red.or.pred q, %1, %2, p;\nselp.u32 %0, 1, 0, q;\n}"
               : "=r"(out) : "r"(id), "r"(nthreads), "r"((uint32_t)flag) : "memory");
  return out != 0;
}

}  // namespace sm100
#endif
