// Temporary: tensor-core paths not built yet.
#include "conv_internal.h"
#include "linear_internal.h"
namespace fth {
bool Tcgen05Supported(int, const LinearArgs&) { return false; }
int LaunchLinearTcgen05(int, const LinearArgs&, const Fp8Epilogue&, const Int8Epilogue&, cudaStream_t) { return FTH_B200_ERR_UNSUPPORTED; }
bool ConvTcgen05Supported(const ConvArgs&) { return false; }
size_t ConvTcgen05WorkspaceBytes(const ConvArgs&) { return 0; }
int LaunchConvTcgen05(const ConvArgs&, cudaStream_t) { return FTH_B200_ERR_UNSUPPORTED; }
}
