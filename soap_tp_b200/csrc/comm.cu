// placeholder until the communicator lands
#include "comm.h"
namespace soapb200 {
void register_comm(pybind11::module_&) {}
}  // namespace soapb200
