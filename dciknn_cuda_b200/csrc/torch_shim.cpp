// PyTorch-extension shim over the C ABI of include/dci_b200.h.
//
// Exposes the seven entry points of the reference's extension module with the
// same names, argument order and return conventions (src/dci_cuda.cpp:175-183:
// _dci_new, _dci_add, _dci_query, _dci_multi_query, _dci_clear, _dci_reset,
// _dci_free), so that the reference's Python layer (dciknn_cuda/core.py) can
// import this module in place of its own `_dci_cuda`.  Everything here is
// tensor plumbing: device guards, output tensors, the caller's current stream;
// the work happens behind the C ABI.
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/dci_b200.h"

namespace py = pybind11;

namespace {

struct Instance {
    dci_b200_t *h = nullptr;
    int device = 0;
    torch::Tensor data;      // keeps the indexed tensor alive: the index borrows its memory (dci_cuda.cpp:80-81)
};

const char *kCapsuleName = "py_dci_inst";   // the reference's capsule name (dci_cuda.cpp:63)

std::atomic<unsigned long long> g_instances{0};

void check(int rc) {
    if (rc == DCI_B200_OK) return;
    const std::string msg = dci_b200_last_error();
    if (rc == DCI_B200_ERR_ARG) throw py::value_error(msg);
    throw std::runtime_error(msg);
}

Instance *unwrap(py::handle capsule) {
    auto *inst = static_cast<Instance *>(PyCapsule_GetPointer(capsule.ptr(), kCapsuleName));
    if (!inst) throw py::error_already_set();
    return inst;
}

Instance *live(py::handle capsule) {
    Instance *inst = unwrap(capsule);
    if (!inst->h) throw std::runtime_error("this DCI instance has been freed");
    return inst;
}

void capsule_destructor(PyObject *capsule) {
    auto *inst = static_cast<Instance *>(PyCapsule_GetPointer(capsule, kCapsuleName));
    if (!inst) return;
    if (inst->h) dci_b200_destroy(inst->h);
    delete inst;
}

// Replaces py_dci_new (dci_cuda.cpp:54-66).  The reference draws directions from the process-global
// rand(); here every instance of a process gets its own seed (DCI_B200_SEED moves the whole sequence).
py::object dci_new(int dim, int num_comp_indices, int num_simp_indices, int device_id) {
    auto *inst = new Instance();
    inst->device = device_id;
    const char *env = std::getenv("DCI_B200_SEED");
    const unsigned long long base = env ? std::strtoull(env, nullptr, 10) : 0ull;
    unsigned long long z = base * 0x9E3779B97F4A7C15ull + (++g_instances) * 0xBF58476D1CE4E5B9ull + 0x94D049BB133111EBull;
    z ^= z >> 31;
    const int rc = dci_b200_create(&inst->h, dim, num_comp_indices, num_simp_indices, device_id, z);
    if (rc) { delete inst; check(rc); }
    return py::reinterpret_steal<py::object>(PyCapsule_New(inst, kCapsuleName, capsule_destructor));
}

void check_tensor(const torch::Tensor &t, const Instance *inst, const char *what) {
    if (!t.is_cuda()) throw py::type_error(std::string(what) + " must be a cuda tensor");
    if (t.scalar_type() != torch::kFloat32) throw py::type_error(std::string(what) + " must consist of single-precision floats");
    if (!t.is_contiguous()) throw py::value_error(std::string(what) + " must be contiguous");
    if (t.get_device() != inst->device) throw py::value_error(std::string(what) + " lives on another device than this DCI instance");
}

// Replaces py_dci_add (dci_cuda.cpp:68-82): py_data is the flattened [num_points, dim] tensor.
void dci_add(py::handle capsule, int dim, int num_points, torch::Tensor py_data, int block_size, int thread_size) {
    Instance *inst = live(capsule);
    check_tensor(py_data, inst, "data");
    if (py_data.numel() != (int64_t)dim * num_points) throw py::value_error("data does not hold num_points x dim values");
    const c10::cuda::CUDAGuard guard(inst->device);
    check(dci_b200_add(inst->h, py_data.data_ptr<float>(), num_points, block_size, thread_size,
                       c10::cuda::getCurrentCUDAStream(inst->device).stream()));
    inst->data = py_data;
}

// Replaces py_dci_query (dci_cuda.cpp:84-118): returns one float32 tensor of 2 * num_queries * k
// values, the neighbour ids (as float32, dci_cuda.cpp:111) followed by the distances (dci_cuda.cpp:115).
torch::Tensor dci_query(py::handle capsule, int dim, int num_queries, torch::Tensor py_query, int num_neighbours, bool blind,
                        int num_outer_iterations, int max_num_candidates, int block_size, int thread_size) {
    Instance *inst = live(capsule);
    check_tensor(py_query, inst, "query");
    if (py_query.numel() != (int64_t)dim * num_queries) throw py::value_error("query does not hold num_queries x dim values");
    if (blind) throw std::runtime_error("blind querying returns lists of another length: use dciknn_cuda_b200.DCI.query(blind=True)");
    const c10::cuda::CUDAGuard guard(inst->device);
    const int64_t n_out = (int64_t)num_queries * num_neighbours;
    auto ids = torch::empty({n_out}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, inst->device));
    auto result = torch::empty({2 * n_out}, torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, inst->device));
    check(dci_b200_query(inst->h, py_query.data_ptr<float>(), num_queries, num_neighbours, num_outer_iterations,
                         max_num_candidates, 0, block_size, thread_size, ids.data_ptr<int>(),
                         result.data_ptr<float>() + n_out, c10::cuda::getCurrentCUDAStream(inst->device).stream()));
    result.narrow(0, 0, n_out).copy_(ids);       // int32 -> float32
    return result;
}

// Replaces py_dci_multi_query (dci_cuda.cpp:120-134).  The reference starts one host thread per
// device because its query blocks; these calls only enqueue work, so one loop keeps all devices busy.
std::vector<torch::Tensor> dci_multi_query(std::vector<py::handle> capsules, int dim, int num_queries,
                                           std::vector<torch::Tensor> py_query, int num_neighbours, bool blind,
                                           int num_outer_iterations, int max_num_candidates, int block_size, int thread_size) {
    if (capsules.size() != py_query.size()) throw py::value_error("one query tensor per DCI instance is needed");
    std::vector<torch::Tensor> results;
    for (size_t i = 0; i < py_query.size(); ++i)
        results.push_back(dci_query(capsules[i], dim, num_queries, py_query[i], num_neighbours, blind, num_outer_iterations,
                                    max_num_candidates, block_size, thread_size));
    return results;
}

void dci_clear(py::handle capsule) {             // replaces py_dci_clear (dci_cuda.cpp:136-147)
    Instance *inst = live(capsule);
    check(dci_b200_clear(inst->h));
    inst->data = torch::Tensor();
}

void dci_reset(py::handle capsule) {             // replaces py_dci_reset (dci_cuda.cpp:149-160): new directions
    Instance *inst = live(capsule);
    unsigned long long z = (++g_instances) * 0xBF58476D1CE4E5B9ull + 0x94D049BB133111EBull;
    z ^= z >> 31;
    check(dci_b200_reset(inst->h, z));
    inst->data = torch::Tensor();
}

void dci_free(py::handle capsule) {              // replaces py_dci_free (dci_cuda.cpp:162-173); freeing twice is harmless
    Instance *inst = unwrap(capsule);
    if (inst->h) dci_b200_destroy(inst->h);
    inst->h = nullptr;
    inst->data = torch::Tensor();
}

// extras for tests: the directions (the reference has no accessor)
torch::Tensor dci_get_proj(py::handle capsule, int rows, int dim) {
    Instance *inst = live(capsule);
    auto out = torch::empty({rows, dim}, torch::kFloat32);
    check(dci_b200_get_proj(inst->h, out.data_ptr<float>()));
    return out;
}

void dci_set_proj(py::handle capsule, torch::Tensor proj) {
    Instance *inst = live(capsule);
    auto p = proj.to(torch::kCPU, torch::kFloat32).contiguous();
    check(dci_b200_set_proj(inst->h, p.data_ptr<float>()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("_dci_new", &dci_new, "Create new DCI instance. (CUDA)");
    m.def("_dci_add", &dci_add, "Add data. (CUDA)");
    m.def("_dci_query", &dci_query, "Search for nearest neighbours. (CUDA)");
    m.def("_dci_clear", &dci_clear, "Clear DCI. (CUDA)");
    m.def("_dci_reset", &dci_reset, "Reset DCI. (CUDA)");
    m.def("_dci_free", &dci_free, "Free DCI. (CUDA)");
    m.def("_dci_multi_query", &dci_multi_query, "Search for nearest neighbours with multiple GPUs. (CUDA)");
    m.def("_dci_get_proj", &dci_get_proj, "Directions as a [rows, dim] CPU tensor.");
    m.def("_dci_set_proj", &dci_set_proj, "Install directions (before add).");
}
