#define FA_INST_HD 256
#define FA_INST_T __half
#define FA_INST_NAME launch_mma_256_fp16
#define FA_INST_CONFIGS FA_MMA_CONFIGS_256
#include "mma_inst.inc"
