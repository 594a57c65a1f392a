#include "symm.h"
void terrace_b200_register_symm(torch::Library& m) { (void)m; }
