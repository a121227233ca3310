// Host-only check of the per-device bookkeeping behind cudaFuncSetAttribute
// (ncnn-moe-runtime_b200/csrc/moe_internal.h): the opt-in for more than 48 KiB
// of dynamic shared memory applies to one device, so what has been configured
// is remembered per device ordinal.  No CUDA call is made.
#include <cstdio>

#include "../../ncnn-moe-runtime_b200/csrc/moe_internal.h"

static int failures = 0;
#define EXPECT(condition)                                              \
    do                                                                 \
    {                                                                  \
        if (!(condition))                                              \
        {                                                              \
            std::printf("line %d: %s\n", __LINE__, #condition);        \
            ++failures;                                                \
        }                                                              \
    } while (0)

int main()
{
    moe::SharedOptIn state;
    EXPECT(moe::opt_in_needed(state, 0, 60000));   // first use on device 0
    EXPECT(!moe::opt_in_needed(state, 0, 60000));  // remembered
    EXPECT(!moe::opt_in_needed(state, 0, 50000));  // a smaller request is covered
    EXPECT(moe::opt_in_needed(state, 0, 100000));  // a larger one is not
    EXPECT(moe::opt_in_needed(state, 1, 60000));   // device 1 has never been configured
    EXPECT(!moe::opt_in_needed(state, 1, 60000));
    EXPECT(!moe::opt_in_needed(state, 0, 100000)); // device 0 keeps its own record
    EXPECT(moe::opt_in_needed(state, moe::kMaxDevices, 1000));  // untracked ordinals configure every time
    EXPECT(moe::opt_in_needed(state, moe::kMaxDevices, 1000));
    EXPECT(moe::opt_in_needed(state, -1, 1000));
    moe::SharedOptIn other;                        // another kernel has its own record
    EXPECT(moe::opt_in_needed(other, 0, 60000));

    // the router's block partition keeps its [expert][block] table within bounds
    for (uint32_t experts : {1u, 256u, 1025u, 4096u})
        for (uint32_t tokens : {1u, 7u, 4096u, 65536u, 1000000u})
        {
            const moe::RouterPartition part = moe::router_partition_host(tokens, experts);
            EXPECT(part.tokens_per_block >= 1 && part.blocks >= 1);
            EXPECT(static_cast<uint64_t>(part.blocks) * part.tokens_per_block >= tokens);
            EXPECT(static_cast<uint64_t>(part.blocks - 1) * part.tokens_per_block < tokens);
            EXPECT(static_cast<uint64_t>(part.blocks) * experts <= MOE_ROUTER_BLOCK_TABLE_ENTRIES);
        }
    if (failures == 0)
        std::puts("opt-in bookkeeping ok");
    return failures == 0 ? 0 : 1;
}
