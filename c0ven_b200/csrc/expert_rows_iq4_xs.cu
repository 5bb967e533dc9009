// k_expert_rows for IQ4_XS weights (expert_rows.cuh).
#define EXPERT_ROWS_QT moe::QT_IQ4_XS
#include "expert_rows_inst.cuh"
