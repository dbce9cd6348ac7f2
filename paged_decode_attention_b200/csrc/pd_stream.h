// Host interface between the C ABI layer (pd_api.cu) and the streaming decode kernel
// (pd_stream.cu).
#pragma once

#include "pd_common.cuh"

namespace pd {

// PD_OK when the streaming kernel serves these (already validated) arguments, else
// PD_ERR_UNSUPPORTED.  Touches no device.
int stream_supports(const PdDecodeArgs* a);

// Scratch the streaming kernel needs for these arguments on a device with `sm_count` SMs.
uint64_t stream_workspace_bytes(const PdDecodeArgs* a, int sm_count);

// Bytes at the start of that scratch that hold the arrival counters of the in-kernel merge.
uint64_t stream_counter_bytes(const PdDecodeArgs* a, int sm_count);

struct PushTargets;

// Launches the streaming decode (which merges its own partial results) on a->stream.  With
// `push`, every finished unit is also stored into the exchange buffers it names.
int stream_run(const PdDecodeArgs* a, Params& p, int sm_count, const PushTargets* push = nullptr);

// Defined in pd_api.cu: argument checks that need no device, the device-side parameter block,
// and the SM count of the current device (or the caller's override).
int validate(const PdDecodeArgs* a, bool need_output = true);
void fill_params(const PdDecodeArgs* a, Params& p);
int resolve_sm_count(const PdDecodeArgs* a);

}  // namespace pd
