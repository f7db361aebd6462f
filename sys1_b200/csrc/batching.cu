// Host-side packing of a ragged batch into the token-packed layout the kernels consume.
// Stands where the reference pads a batch to [batch, max_len] (src/models/laya.rs:396-431) after its batcher
// has grouped requests by count (src/batching.rs:83-102); the offsets have the shape the reference builds for
// its varlen attention path (src/archs/modernbert.rs:431-443).
#include <stdint.h>

#include "../../include/sys1_b200.h"

extern "C" int s1_pack_batch(const int32_t* lengths_host, int num_sequences, int token_budget, int pad_multiple,
                             int32_t* cu_seqlens_host, int32_t* positions_host, int* num_taken, int* total_tokens,
                             int* padded_tokens) {
    if (!lengths_host || !cu_seqlens_host || !num_taken || !total_tokens || !padded_tokens) return S1_EINVAL;
    if (num_sequences < 0 || token_budget < 1 || pad_multiple < 1) return S1_EINVAL;
    long long total = 0;
    int taken = 0;
    cu_seqlens_host[0] = 0;
    for (int i = 0; i < num_sequences; ++i) {
        const int len = lengths_host[i];
        if (len < 0) return S1_EINVAL;
        // a sequence longer than the budget is a batch of its own
        if (taken > 0 && total + len > token_budget) break;
        if (total + len > INT32_MAX) return S1_EINVAL;
        if (positions_host) {
            for (int t = 0; t < len; ++t) positions_host[total + t] = t;
        }
        total += len;
        ++taken;
        cu_seqlens_host[taken] = static_cast<int32_t>(total);
        if (total >= token_budget) break;
    }
    *num_taken = taken;
    *total_tokens = static_cast<int>(total);
    *padded_tokens = static_cast<int>((total + pad_multiple - 1) / pad_multiple * pad_multiple);
    return S1_OK;
}
