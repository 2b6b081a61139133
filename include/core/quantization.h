/* C-ML's include/core/quantization.h, served by libcml_b200: the int8 / uint8 / NF4 quantisers are declared in cml_quant_api.h. */
#ifndef CML_B200_CORE_QUANTIZATION_H
#define CML_B200_CORE_QUANTIZATION_H
#include "../cml_quant_api.h"
#endif
