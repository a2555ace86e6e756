// Internal declarations shared by the translation units of the device library.
#pragma once
#include "common.cuh"

// Drops the digit-pass events collected for the context's device.
void sort_reset_timing(csa_ctx* ctx);
