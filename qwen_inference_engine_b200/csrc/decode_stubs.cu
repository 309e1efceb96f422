// decode_stubs.cu -- stands in for decode_mega.cu and decode_gemv.cu (the Qwen family's two persistent decode kernels,
// by far the longest compiles of the library) in libqie_b200_lean.so: both report that they support no shape, so the
// engine takes its per-operator decode path.  Everything else -- every family's forward, cache and state manager,
// scheduler, C ABI -- is the same code as in the full library.  bin/trace_run builds and loads the lean library.
#include "kernels.h"

namespace qie {

int decode_mega_kc(int, int) { return 64; }
bool decode_mega_supports(int, int, int, int, int, int, int, int, int, int, int, int) { return false; }
int decode_mega_prof_slots(int) { return 1; }
cudaError_t launch_decode_mega(MegaArgs, int, cudaStream_t) { return cudaErrorNotSupported; }
bool decode_gemv_supports(int, int, int, int, int, int, int, int, int) { return false; }
size_t decode_gemv_scratch_bytes(int, int, int, int, int, int, int) { return 16; }
cudaError_t launch_decode_gemv(MegaArgs, void*, int, cudaStream_t, int) { return cudaErrorNotSupported; }

}  // namespace qie
