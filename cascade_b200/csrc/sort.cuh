// Internal declarations shared by the translation units of the device library.
#pragma once
#include "common.cuh"

// Drops the digit-pass events collected for the context's device.
void sort_reset_timing(csa_ctx* ctx);
// Frees the context's digit-pass timer.
void sort_free_timing(csa_ctx* ctx);

// Device address of the digit histograms ([pass][256] 64-bit counts) left in the workspace by the last csa_sort_pairs of n records.
const u64* sort_workspace_histograms(void* workspace, size_t workspace_bytes, u64 n);

// Test hook of the part-at-a-time build: the offset added to every position that is put into a lane.
void stream_set_position_offset(u64 offset);
