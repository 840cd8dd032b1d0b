// Symmetric-memory communicator: bindings registered by comm.cu.
#pragma once
#include <pybind11/pybind11.h>

namespace soapb200 {
void register_comm(pybind11::module_& m);
}
