// XLA-FFI handlers over the C ABI (include/ragged_dot_b200.h), for use as jax.ffi custom calls.
//
// Compiled only where jaxlib's FFI headers exist:
//   g++ -shared -fPIC -std=c++17 -I$(python -c "import jax; print(jax.ffi.include_dir())") \
//       -I/usr/local/cuda/include xla_ffi_shim.cc -L.. -l:librd_b200.so -o librd_b200_xla.so
// Without those headers this file compiles to nothing.  The handlers add no logic: they unpack
// buffers, call rd_gmm / rd_tgmm on XLA's stream and map a non-zero status to an ffi::Error.
// The workspace is an extra result buffer so the handlers never allocate.
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define RD_HAVE_XLA_FFI 1
#endif
#endif

#ifdef RD_HAVE_XLA_FFI
#include <cuda_runtime_api.h>

#include "../../include/ragged_dot_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int DtypeCode(ffi::DataType t) {
  if (t == ffi::DataType::BF16) return RD_DTYPE_BF16;
  if (t == ffi::DataType::F16) return RD_DTYPE_F16;
  if (t == ffi::DataType::F32) return RD_DTYPE_F32;  // multiplied as TF32, float32 result
  return -1;
}

ffi::Error ToError(int rc, const char* where) {
  if (rc == RD_OK) return ffi::Error::Success();
  return ffi::Error(rc == RD_ERR_LAUNCH || rc == RD_ERR_DRIVER ? ffi::ErrorCode::kInternal
                                                               : ffi::ErrorCode::kInvalidArgument,
                    std::string(where) + ": " + rd_status_string(rc));
}

ffi::Error GmmImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer a,
                   ffi::Buffer<ffi::S32> group_sizes, ffi::Result<ffi::AnyBuffer> y,
                   ffi::Result<ffi::AnyBuffer> workspace, bool trans_rhs, int32_t tile_n) {
  auto xd = x.dimensions();
  auto ad = a.dimensions();
  if (xd.size() != 2 || ad.size() != 3 || group_sizes.dimensions().size() != 1 ||
      ad[0] != group_sizes.dimensions()[0])
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "rd_gmm: expected x[m,k], A[g,.,.], gs[g]");
  const int m = static_cast<int>(xd[0]), k = static_cast<int>(xd[1]), g = static_cast<int>(ad[0]);
  const int n = static_cast<int>(trans_rhs ? ad[1] : ad[2]);
  rd_tile_cfg cfg{tile_n, 0, 0, 0, 0, 0};
  return ToError(rd_gmm(x.untyped_data(), a.untyped_data(), group_sizes.typed_data(),
                        y->untyped_data(), workspace->untyped_data(), workspace->size_bytes(), m, k, n,
                        g, trans_rhs ? 1 : 0, DtypeCode(x.element_type()), tile_n ? &cfg : nullptr,
                        stream),
                 "rd_gmm");
}

ffi::Error TgmmImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer dout,
                    ffi::Buffer<ffi::S32> group_sizes, ffi::Result<ffi::AnyBuffer> out,
                    ffi::Result<ffi::AnyBuffer> workspace, int32_t tile_n) {
  auto xd = x.dimensions();
  auto dd = dout.dimensions();
  if (xd.size() != 2 || dd.size() != 2 || xd[0] != dd[0])
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "rd_tgmm: expected x[m,k], dout[m,n]");
  const int m = static_cast<int>(xd[0]), k = static_cast<int>(xd[1]), n = static_cast<int>(dd[1]);
  const int g = static_cast<int>(group_sizes.dimensions()[0]);
  rd_tile_cfg cfg{tile_n, 0, 0, 0, 0, 0};
  return ToError(rd_tgmm(x.untyped_data(), dout.untyped_data(), group_sizes.typed_data(),
                         out->untyped_data(), workspace->untyped_data(), workspace->size_bytes(), m, k,
                         n, g, DtypeCode(x.element_type()), tile_n ? &cfg : nullptr, stream),
                 "rd_tgmm");
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(RdGmmFfi, GmmImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<bool>("trans_rhs")
                                  .Attr<int32_t>("tile_n"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(RdTgmmFfi, TgmmImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("tile_n"));
#endif  // RD_HAVE_XLA_FFI
