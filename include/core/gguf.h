/* C-ML's include/core/gguf.h, served by libcml_b200: the GGUF reader is declared in cml_quant_api.h (reading only: C-ML's writer cannot emit quantized tensors). */
#ifndef CML_B200_CORE_GGUF_H
#define CML_B200_CORE_GGUF_H
#include "../cml_quant_api.h"
#endif
