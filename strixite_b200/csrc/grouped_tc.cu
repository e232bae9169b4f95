// tcgen05 grouped expert GEMMs (placeholder translation unit while the kernels are brought up).
#include "experts.cuh"

namespace sxb {

template <int BITS>
int tc_gather_grouped(const char *fn, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t, void *,
                      int, bool, bool, sxb_stream_t) {
    SXB_CHECK(false, fn, ": the WMMA_F16 (tcgen05) kernels are not built into this library");
    return SXB_OK;
}
template <int BITS>
int tc_partial_grouped(const char *fn, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t, float *,
                       int, bool, sxb_stream_t) {
    SXB_CHECK(false, fn, ": the WMMA_F16 (tcgen05) kernels are not built into this library");
    return SXB_OK;
}
template int tc_gather_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, bool, sxb_stream_t);
template int tc_gather_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                  void *, int, bool, bool, sxb_stream_t);
template int tc_partial_grouped<4>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, bool, sxb_stream_t);
template int tc_partial_grouped<8>(const char *, const void *, const SxbQView *, int64_t, const void *, size_t, int64_t, int64_t,
                                   float *, int, bool, sxb_stream_t);

}  // namespace sxb
