// Temporary: tensor-core paths not built yet.
#include "conv_internal.h"
namespace fth {
bool ConvTcgen05Supported(const ConvArgs&) { return false; }
size_t ConvTcgen05WorkspaceBytes(const ConvArgs&) { return 0; }
int LaunchConvTcgen05(const ConvArgs&, cudaStream_t) { return FTH_B200_ERR_UNSUPPORTED; }
}
