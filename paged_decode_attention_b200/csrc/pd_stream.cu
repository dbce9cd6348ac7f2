#include "pd_stream.h"
namespace pd {
int stream_supports(const PdDecodeArgs*) { return PD_ERR_UNSUPPORTED; }
uint64_t stream_workspace_bytes(const PdDecodeArgs*, int) { return 0; }
int stream_run(const PdDecodeArgs*, Params&, int) { return PD_ERR_UNSUPPORTED; }
}
