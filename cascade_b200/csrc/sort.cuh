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

// Sorts the segments [seg_off_host[s], seg_off_host[s + 1]) of one record array, each on its own, in one set of launches and
// without a read-back; every pass runs, so the records end in the alt buffers iff the number of passes is odd. Values are
// 32-bit (or absent: both pointers null). Every segment holds fewer than 2^30 records.
size_t sort_segments_workspace_bytes(u64 n, u32 segs);
int sort_segments(csa_ctx* ctx, u64* keys, u64* keys_alt, u32* vals, u32* vals_alt, const u64* seg_off_host, u32 segs, int begin_bit, int end_bit, void* workspace,
                  size_t workspace_bytes, int* in_alt);
