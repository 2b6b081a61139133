/* C-ML's include/core/gguf_quant.h, served by libcml_b200: the block types and their dequantisers are declared in cml_quant_api.h. */
#ifndef CML_B200_CORE_GGUF_QUANT_H
#define CML_B200_CORE_GGUF_QUANT_H
#include "../cml_quant_api.h"
#endif
