/* C-ML's include/nn/lora.h, served by libcml_b200: the LoRA layer and adapter are declared in cml_quant_api.h. */
#ifndef CML_B200_NN_LORA_H
#define CML_B200_NN_LORA_H
#include "../cml_quant_api.h"
#endif
