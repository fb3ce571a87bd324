#define FTA_INST_D 64
#include "fta_stage1_mma_inst.inc"
