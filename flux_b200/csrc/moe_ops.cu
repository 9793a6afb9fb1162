// MoE grouped ops (placeholder while the dense path is brought up).
#include "internal.h"
using namespace fluxb;
extern "C" {
size_t fluxb_moe_ag_scatter_workspace_bytes(int, int, int) { return 0; }
int fluxb_moe_ag_scatter_create(fluxb_comm_t, int, int, int, int, int, int, int, void* const*, int* const*, void*, fluxb_moe_ag_scatter_t*) { FLUXB_FAIL(FLUXB_ERR_UNSUPPORTED, "not built yet"); }
int fluxb_moe_ag_scatter_destroy(fluxb_moe_ag_scatter_t) { return FLUXB_OK; }
int fluxb_moe_ag_scatter_forward(fluxb_moe_ag_scatter_t, const void*, int, const void*, const int*, const int*, const float*, void*, void*, const fluxb_tuning*, fluxb_stream_t) { FLUXB_FAIL(FLUXB_ERR_UNSUPPORTED, "not built yet"); }
size_t fluxb_moe_gather_rs_workspace_bytes(int, int, int, int) { return 0; }
size_t fluxb_moe_gather_rs_stage_bytes(int, int, int, int) { return 0; }
size_t fluxb_moe_gather_rs_cnt_bytes(int, int, int) { return 0; }
int fluxb_moe_gather_rs_create(fluxb_comm_t, int, int, int, int, int, int, float* const*, int* const*, void*, fluxb_moe_gather_rs_t*) { FLUXB_FAIL(FLUXB_ERR_UNSUPPORTED, "not built yet"); }
int fluxb_moe_gather_rs_destroy(fluxb_moe_gather_rs_t) { return FLUXB_OK; }
int fluxb_moe_gather_rs_forward(fluxb_moe_gather_rs_t, const void*, int, int, const void*, const int*, const int*, const float*, const float*, const float*, void*, const fluxb_tuning*, fluxb_stream_t) { FLUXB_FAIL(FLUXB_ERR_UNSUPPORTED, "not built yet"); }
}
