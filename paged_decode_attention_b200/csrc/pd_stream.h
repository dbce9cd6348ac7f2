// Host interface of the streaming decode kernel (pd_stream.cu) used by the C ABI layer.
#pragma once

#include "pd_common.cuh"

namespace pd {

// PD_OK when the streaming kernel serves these (already validated) arguments, else
// PD_ERR_UNSUPPORTED.  Touches no device.
int stream_supports(const PdDecodeArgs* a);

// Scratch the streaming kernel needs for these arguments on a device with `sm_count` SMs.
uint64_t stream_workspace_bytes(const PdDecodeArgs* a, int sm_count);

// Launches the streaming decode and its merge on a->stream.
int stream_run(const PdDecodeArgs* a, Params& p, int sm_count);

}  // namespace pd
