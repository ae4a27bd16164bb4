// NOT onnx-light: forwards to the stand-in used where onnx-light is not installed.
#pragma once
#include "onnx_core/onnx_light_shim.h"
