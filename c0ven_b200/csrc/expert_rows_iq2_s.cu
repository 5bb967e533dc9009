// k_expert_rows for IQ2_S weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_IQ2_S
#include "expert_rows_inst.cuh"
