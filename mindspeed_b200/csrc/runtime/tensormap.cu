// Host-side construction of TMA tensor maps. The driver entry point is resolved at run time through the CUDA
// runtime, so the library has no link-time dependency on libcuda.
#include "msb_common.cuh"
#include "msb_sm100.cuh"
#include <mutex>

namespace msb {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_encodeTiled)p;
  });
  return fn;
}

// The encode call is a driver entry point: it needs a context current on the calling thread, but a thread whose first
// CUDA work is this call (an autograd worker thread running a GEMM as its first backward node on device 0) has none yet,
// because only runtime calls bind the primary context lazily.  One runtime call per thread does that.
static inline void ensure_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) { msb_set_error("cuTensorMapEncodeTiled is not available from this driver"); return 1; }
  ensure_context();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) { msb_set_error("tensor map base %p is not 16-byte aligned", base); return 2; }
  if ((ld * elem_bytes) % 16 != 0) { msb_set_error("tensor map row pitch %llu bytes is not a multiple of 16", (unsigned long long)(ld * elem_bytes)); return 2; }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = (box_cols * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (box_cols * elem_bytes == 64) ? CU_TENSOR_MAP_SWIZZLE_64B
                          : (box_cols * elem_bytes == 32) ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msb_set_error("cuTensorMapEncodeTiled failed (%d) rows=%llu cols=%llu ld=%llu box=%ux%u", (int)r, (unsigned long long)rows,
                  (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols);
    return 1;
  }
  return 0;
}

int make_tmap_nd(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) { msb_set_error("cuTensorMapEncodeTiled is not available from this driver"); return 1; }
  ensure_context();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) { msb_set_error("tensor map base %p is not 16-byte aligned", base); return 2; }
  cuuint64_t gdim[5]; cuuint64_t gstr[4]; cuuint32_t bx[5]; cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] % 16 != 0) { msb_set_error("tensor map stride %llu is not a multiple of 16 bytes", (unsigned long long)strides_bytes[i]); return 2; }
    gstr[i] = strides_bytes[i];
  }
  const uint32_t inner = box[0] * (uint32_t)elem_bytes;
  CUtensorMapSwizzle sw = inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : inner == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { msb_set_error("cuTensorMapEncodeTiled (rank %d) failed (%d)", rank, (int)r); return 1; }
  return 0;
}

}  // namespace msb
