// What the expert-parallel wrapper (ep.cu) needs from the layer object beyond the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "infmoe_c.h"

namespace infmoe {

// The experts of `layer` applied to rows that sit in the slots of a partly filled buffer: `slots` slots in regions
// of region_size, of which the first d_region_count[s] of region s hold a row; d_expert_of_slot gives the expert of
// every filled slot.  The result of slot i is written to the address d_slot_dst[i]; with d_slot_score the
// base_layer output mix is applied on the way.  Stream ordered, no host synchronisation when the experts are
// resident.  Workspace as for infmoe_layer_enqueue with token_num = slots.
int layer_run_slots(infmoe_layer* layer, const float* d_rows, const int32_t* d_expert_of_slot,
                    const float* d_slot_score, const unsigned long long* d_slot_dst, void* d_workspace,
                    size_t workspace_bytes, int64_t slots, const int32_t* d_region_count, int32_t region_size,
                    cudaStream_t stream);

// Copies the layer's device status word into *h_word (page-locked) and clears it, stream ordered, without waiting;
// layer_status_code turns such a word into the return code infmoe_layer_sync_status would give.
int layer_snapshot_status(infmoe_layer* layer, int* h_word, cudaStream_t stream);
int layer_status_code(int word);

}  // namespace infmoe
