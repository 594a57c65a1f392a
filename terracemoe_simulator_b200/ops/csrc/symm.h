// Registration hook of the symmetric-memory runtime ops (symm_bindings.cpp).
#pragma once
#include <torch/library.h>

void terrace_b200_register_symm(torch::Library& m);
void terrace_b200_register_symm_cuda(torch::Library& m);
