#define FTA_INST_D 128
#include "fta_stage1_mma_inst.inc"
