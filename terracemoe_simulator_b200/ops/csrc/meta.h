// Registration hook of the shape-only (Meta) implementations (meta_bindings.cpp).
#pragma once
#include <torch/library.h>

void terrace_b200_register_meta(torch::Library& m);
