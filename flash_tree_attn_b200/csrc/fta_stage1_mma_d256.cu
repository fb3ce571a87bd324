#define FTA_INST_D 256
#include "fta_stage1_mma_inst.inc"
