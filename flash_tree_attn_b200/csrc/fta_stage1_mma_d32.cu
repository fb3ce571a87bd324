#define FTA_INST_D 32
#include "fta_stage1_mma_inst.inc"
