// Python module inside the host library (imported by torch_supa_b200.distributed as `_supa_c10d`): the creator function
// torch.distributed.Backend.register_backend needs, which returns the c10d backend for supa tensors.
#include <pybind11/chrono.h>
#include <torch/csrc/utils/pybind.h>

#include "SupaBackend.h"

PYBIND11_MODULE(_supa_c10d, m) {
  m.doc() = "c10d backend for the supa device (NCCL underneath)";
  m.def(
      "create_backend",
      [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, const std::chrono::milliseconds& timeout) {
        return supa::create_supa_backend(store, rank, size, timeout);
      },
      py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"), py::call_guard<py::gil_scoped_release>());
}
