/* C-ML's include/nn/qlora.h, served by libcml_b200: the NF4 tensor and the QLoRA linear are declared in cml_quant_api.h. */
#ifndef CML_B200_NN_QLORA_H
#define CML_B200_NN_QLORA_H
#include "../cml_quant_api.h"
#endif
