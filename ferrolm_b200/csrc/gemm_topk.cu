// placeholder for the tensor-core front end; replaced by the tcgen05 implementation
#include "internal.h"
namespace fv {
struct TcSide {};
void tc_free(TcSide* tc) { delete tc; }
int tc_append(fv_ctx*, TcSide**, int, const float*, size_t, size_t, int) { return FV_OK; }
int tc_search(fv_ctx*, TcSide*, int, const float*, size_t, int, const float*, size_t, int, uint32_t, u64*) {
  return fail(FV_ERR_UNSUPPORTED, "tensor-core search is not built");
}
bool tc_usable(const TcSide*, size_t, size_t, int) { return false; }
}  // namespace fv
