// PJRT C-API entry of the B200 build: the C++ front door that stands where the reference's
// `plugin/metal_pjrt.cc` stands. Like it, this is a thin shim: jaxlib (or any PJRT host) loads
// the shared object, calls `GetPjrtApi()` (plugin/metal_pjrt.cc:1276), and every compile /
// execute / transfer re-enters the Python engine (`metaljax_b200.engine`) under the GIL, where
// the quantized-matmul recognizer rewrites the matched dots into calls of libqmm. One device
// (the current CUDA device), one memory space, every event born ready, everything synchronous
// (plugin/metal_pjrt.cc:55-57, 416-432, 478-482).
//
// Implemented: the same subset the reference implements (plugin/metal_pjrt.cc:1288-1411) --
// Error_*, Plugin_*, Event_*, Client_{Create, Destroy, PlatformName, ProcessIndex,
// PlatformVersion, Devices, AddressableDevices, LookupDevice, LookupAddressableDevice,
// AddressableMemories, Compile, DefaultDeviceAssignment, BufferFromHostBuffer},
// DeviceDescription_*, Device_*, Memory_*, Executable_*, LoadedExecutable_{Destroy,
// GetExecutable, AddressableDevices, Delete, IsDeleted, Execute, Fingerprint}, Buffer_{Destroy,
// ElementType, Dimensions, UnpaddedDimensions, DynamicDimensionIndices, OnDeviceSizeInBytes,
// Device, Memory, Delete, IsDeleted, CopyToDevice, ToHostBuffer, IsOnCpu, ReadyEvent,
// UnsafePointer}. Every other entry of the table returns PJRT_Error_Code_UNIMPLEMENTED with
// its own name in the message (plugin/metal_pjrt.cc:1199-1262).
//
// Errors: a Python exception becomes a PJRT_Error carrying "Type: message"; a class whose name
// contains "Unsupported" maps to UNIMPLEMENTED, ValueError / TypeError to INVALID_ARGUMENT,
// everything else to INTERNAL (plugin/metal_pjrt.cc:185-226).
//
// When the host process has no Python interpreter yet (a C++ host), the plugin starts one:
// QMM_PJRT_PYTHON names the interpreter whose environment (site-packages) to use, default
// `python3` on PATH; the package is found next to this shared object (<root>/plugin/ -> <root>).
#include <Python.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "pjrt_c_api.h"

namespace {

// ---------------------------------------------------------------- objects

struct QmmError : PJRT_Error {
  std::string message;
  PJRT_Error_Code code;
};

void ErrDestroy(PJRT_Error* e) { delete static_cast<QmmError*>(e); }
void ErrMessage(const PJRT_Error* e, const char** m, size_t* n) {
  const auto* q = static_cast<const QmmError*>(e);
  *m = q->message.c_str();
  *n = q->message.size();
}
PJRT_Error_Code ErrCode(const PJRT_Error* e) { return static_cast<const QmmError*>(e)->code; }
void ErrPayloads(const PJRT_Error*, PJRT_Error_PayloadVisitor, void*) {}

const PJRT_Error_FunctionTable kErrorTable = {
    PJRT_Error_FunctionTable_STRUCT_SIZE, sizeof(QmmError), nullptr, ErrDestroy, ErrMessage, ErrCode, ErrPayloads,
};

PJRT_Error* MakeError(PJRT_Error_Code code, const std::string& msg) {
  auto* e = new QmmError;
  e->vtable = &kErrorTable;
  e->message = msg;
  e->code = code;
  return e;
}

std::mutex g_user_data_mu;
std::map<const void*, std::pair<void*, void (*)(void*)>> g_user_data;
void* MemGetUserData(PJRT_Memory*, const void* key) {
  std::lock_guard<std::mutex> lock(g_user_data_mu);
  auto it = g_user_data.find(key);
  return it == g_user_data.end() ? nullptr : it->second.first;
}
void MemSetUserData(PJRT_Memory*, const void* key, void* data, void (*dtor)(void*)) {
  std::lock_guard<std::mutex> lock(g_user_data_mu);
  auto& slot = g_user_data[key];
  if (slot.first && slot.second) slot.second(slot.first);
  slot = {data, dtor};
}
const PJRT_Memory_FunctionTable kMemoryTable = {
    PJRT_Memory_FunctionTable_STRUCT_SIZE, nullptr, sizeof(PJRT_Memory), MemGetUserData, MemSetUserData,
};

}  // namespace

struct PJRT_Event {
  PJRT_Error* error = nullptr;   // owned; null = success. Always ready.
};
struct PJRT_DeviceDescription {};
struct PJRT_Device {};
struct PJRT_Client {};

struct PJRT_Executable {
  PyObject* program = nullptr;   // owned: metaljax_b200.engine.Program
  int refs = 1;
  std::string name, fingerprint;
  size_t num_outputs = 0;
  std::vector<PJRT_Buffer_Type> out_types;
  std::vector<int64_t> flat_dims;
  std::vector<size_t> dim_sizes;
  std::vector<const char*> memory_kinds;
  std::vector<size_t> memory_kind_sizes;
  std::vector<int64_t> donated;
};
struct PJRT_LoadedExecutable {
  PJRT_Executable* exec = nullptr;
  bool deleted = false;
};
struct PJRT_Buffer {
  PyObject* py = nullptr;        // owned: engine.DeviceBuffer (.data, .type_enum, .dims, .nbytes)
  PJRT_Buffer_Type type = PJRT_Buffer_Type_INVALID;
  std::vector<int64_t> dims;
  size_t nbytes = 0;
  bool deleted = false;
};

namespace {

PJRT_DeviceDescription g_desc;
PJRT_Device g_device;
PJRT_Memory g_memory = {&kMemoryTable};
PJRT_Device* g_devices[1] = {&g_device};
PJRT_Memory* g_memories[1] = {&g_memory};
PJRT_Client g_client;
PyObject* g_engine = nullptr;
std::string g_device_kind = "NVIDIA GPU";
const char kMemoryKind[] = "device";
const char kPlatform[] = "qmm_b200";
const char kPlatformVersion[] = "metaljax-b200 0.1 (PJRT C API " "0.114" ")";
std::once_flag g_python_once;
std::string g_python_error;

class Gil {
 public:
  Gil() : state_(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(state_); }
 private:
  PyGILState_STATE state_;
};

// The pending Python exception as a PJRT_Error (and cleared).
PJRT_Error* PyErrToErr(const char* where) {
  PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  std::string cls = "Exception", msg;
  if (type) {
    PyObject* n = PyObject_GetAttrString(type, "__name__");
    if (n) {
      const char* s = PyUnicode_AsUTF8(n);
      if (s) cls = s;
      Py_DECREF(n);
    }
  }
  if (value) {
    PyObject* s = PyObject_Str(value);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) msg = c;
      Py_DECREF(s);
    }
  }
  PyErr_Clear();
  Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(tb);
  PJRT_Error_Code code = PJRT_Error_Code_INTERNAL;
  if (cls.find("Unsupported") != std::string::npos || cls == "NotImplementedError") code = PJRT_Error_Code_UNIMPLEMENTED;
  else if (cls == "ValueError" || cls == "TypeError") code = PJRT_Error_Code_INVALID_ARGUMENT;
  return MakeError(code, std::string(where) + ": " + cls + ": " + msg);
}

std::string ThisLibraryDir() {
  Dl_info info;
  if (!dladdr(reinterpret_cast<void*>(&ThisLibraryDir), &info) || !info.dli_fname) return ".";
  std::string path = info.dli_fname;
  const size_t slash = path.rfind('/');
  return slash == std::string::npos ? "." : path.substr(0, slash);
}

std::string FindOnPath(const char* name) {
  if (strchr(name, '/')) return name;
  const char* path = getenv("PATH");
  if (!path) return name;
  std::string p = path;
  size_t start = 0;
  while (start <= p.size()) {
    size_t end = p.find(':', start);
    if (end == std::string::npos) end = p.size();
    const std::string cand = p.substr(start, end - start) + "/" + name;
    if (access(cand.c_str(), X_OK) == 0) return cand;
    start = end + 1;
  }
  return name;
}

// Starts an interpreter when the host has none, then imports the engine.
void StartPython() {
  if (!Py_IsInitialized()) {
    PyConfig config;
    PyConfig_InitPythonConfig(&config);
    const char* exe = getenv("QMM_PJRT_PYTHON");
    const std::string path = FindOnPath(exe && *exe ? exe : "python3");
    PyStatus st = PyConfig_SetBytesString(&config, &config.executable, path.c_str());      // finds the venv's pyvenv.cfg
    if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.program_name, path.c_str());
    if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
    PyConfig_Clear(&config);
    if (PyStatus_Exception(st)) {
      g_python_error = std::string("could not start Python: ") + (st.err_msg ? st.err_msg : "?");
      return;
    }
    PyEval_SaveThread();           // release the GIL the initializing thread holds
  }
  Gil gil;
  const std::string root = ThisLibraryDir() + "/..";
  PyObject* sys_path = PySys_GetObject("path");   // borrowed
  if (sys_path) {
    PyObject* r = PyUnicode_FromString(root.c_str());
    if (r) {
      PyList_Insert(sys_path, 0, r);
      Py_DECREF(r);
    }
  }
  g_engine = PyImport_ImportModule("metaljax_b200.engine");
  if (!g_engine) {
    PJRT_Error* e = PyErrToErr("import metaljax_b200.engine");
    g_python_error = static_cast<QmmError*>(e)->message;
    ErrDestroy(e);
    return;
  }
  PyObject* kind = PyObject_CallMethod(g_engine, "device_kind", nullptr);
  if (kind) {
    const char* s = PyUnicode_AsUTF8(kind);
    if (s) g_device_kind = s;
    Py_DECREF(kind);
  } else {
    PyErr_Clear();
  }
}

PJRT_Error* EnsureEngine() {
  std::call_once(g_python_once, StartPython);
  if (!g_engine) return MakeError(PJRT_Error_Code_FAILED_PRECONDITION, g_python_error.empty() ? "engine not loaded" : g_python_error);
  return nullptr;
}

PJRT_Event* ReadyEvent() { return new PJRT_Event; }

// Reads .type_enum / .dims / .nbytes of an engine buffer into a PJRT_Buffer that owns it.
PJRT_Buffer* WrapBuffer(PyObject* py /* stolen */) {
  auto* b = new PJRT_Buffer;
  b->py = py;
  PyObject* t = PyObject_GetAttrString(py, "type_enum");
  if (t) { b->type = static_cast<PJRT_Buffer_Type>(PyLong_AsLong(t)); Py_DECREF(t); }
  PyObject* d = PyObject_GetAttrString(py, "dims");
  if (d) {
    const Py_ssize_t n = PySequence_Size(d);
    for (Py_ssize_t i = 0; i < n; ++i) {
      PyObject* it = PySequence_GetItem(d, i);
      b->dims.push_back(PyLong_AsLongLong(it));
      Py_XDECREF(it);
    }
    Py_DECREF(d);
  }
  PyObject* nb = PyObject_GetAttrString(py, "nbytes");
  if (nb) { b->nbytes = PyLong_AsSize_t(nb); Py_DECREF(nb); }
  PyErr_Clear();
  return b;
}

bool ReadIntList(PyObject* obj, const char* attr, std::vector<int64_t>* out) {
  PyObject* seq = PyObject_GetAttrString(obj, attr);
  if (!seq) return false;
  const Py_ssize_t n = PySequence_Size(seq);
  for (Py_ssize_t i = 0; i < n; ++i) {
    PyObject* it = PySequence_GetItem(seq, i);
    out->push_back(PyLong_AsLongLong(it));
    Py_XDECREF(it);
  }
  Py_DECREF(seq);
  return !PyErr_Occurred();
}

bool ReadString(PyObject* obj, const char* attr, std::string* out) {
  PyObject* s = PyObject_GetAttrString(obj, attr);
  if (!s) return false;
  const char* c = PyUnicode_AsUTF8(s);
  if (c) *out = c;
  Py_DECREF(s);
  return c != nullptr;
}

// ---------------------------------------------------------------- errors, plugin, events

void Error_Destroy(PJRT_Error_Destroy_Args* a) { if (a->error) a->error->vtable->destroy(a->error); }
void Error_Message(PJRT_Error_Message_Args* a) { a->error->vtable->message(a->error, &a->message, &a->message_size); }
PJRT_Error* Error_GetCode(PJRT_Error_GetCode_Args* a) { a->code = a->error->vtable->get_code(a->error); return nullptr; }

PJRT_Error* Plugin_Initialize(PJRT_Plugin_Initialize_Args*) { return nullptr; }   // the engine loads with the first client
PJRT_Error* Plugin_Attributes(PJRT_Plugin_Attributes_Args* a) {
  a->attributes = nullptr;
  a->num_attributes = 0;
  return nullptr;
}

PJRT_Error* Event_Destroy(PJRT_Event_Destroy_Args* a) {
  if (a->event) {
    if (a->event->error) ErrDestroy(a->event->error);
    delete a->event;
  }
  return nullptr;
}
PJRT_Error* Event_IsReady(PJRT_Event_IsReady_Args* a) { a->is_ready = true; return nullptr; }
PJRT_Error* CloneError(const PJRT_Error* e) {
  const auto* q = static_cast<const QmmError*>(e);
  return MakeError(q->code, q->message);
}
PJRT_Error* Event_Error(PJRT_Event_Error_Args* a) { return a->event->error ? CloneError(a->event->error) : nullptr; }
PJRT_Error* Event_Await(PJRT_Event_Await_Args* a) { return a->event->error ? CloneError(a->event->error) : nullptr; }
PJRT_Error* Event_OnReady(PJRT_Event_OnReady_Args* a) {
  a->callback(a->event->error ? CloneError(a->event->error) : nullptr, a->user_arg);    // already ready: call now
  return nullptr;
}

// ---------------------------------------------------------------- client, device, memory

PJRT_Error* Client_Create(PJRT_Client_Create_Args* a) {
  if (PJRT_Error* e = EnsureEngine()) return e;
  a->client = &g_client;
  return nullptr;
}
PJRT_Error* Client_Destroy(PJRT_Client_Destroy_Args*) { return nullptr; }
PJRT_Error* Client_PlatformName(PJRT_Client_PlatformName_Args* a) {
  a->platform_name = kPlatform;
  a->platform_name_size = sizeof(kPlatform) - 1;
  return nullptr;
}
PJRT_Error* Client_ProcessIndex(PJRT_Client_ProcessIndex_Args* a) { a->process_index = 0; return nullptr; }
PJRT_Error* Client_PlatformVersion(PJRT_Client_PlatformVersion_Args* a) {
  a->platform_version = kPlatformVersion;
  a->platform_version_size = sizeof(kPlatformVersion) - 1;
  return nullptr;
}
PJRT_Error* Client_Devices(PJRT_Client_Devices_Args* a) { a->devices = g_devices; a->num_devices = 1; return nullptr; }
PJRT_Error* Client_AddressableDevices(PJRT_Client_AddressableDevices_Args* a) {
  a->addressable_devices = g_devices;
  a->num_addressable_devices = 1;
  return nullptr;
}
PJRT_Error* Client_LookupDevice(PJRT_Client_LookupDevice_Args* a) {
  if (a->id != 0) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "there is one device, id 0");
  a->device = &g_device;
  return nullptr;
}
PJRT_Error* Client_LookupAddressableDevice(PJRT_Client_LookupAddressableDevice_Args* a) {
  if (a->local_hardware_id != 0) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "there is one device, id 0");
  a->addressable_device = &g_device;
  return nullptr;
}
PJRT_Error* Client_AddressableMemories(PJRT_Client_AddressableMemories_Args* a) {
  a->addressable_memories = g_memories;
  a->num_addressable_memories = 1;
  return nullptr;
}
PJRT_Error* Client_DefaultDeviceAssignment(PJRT_Client_DefaultDeviceAssignment_Args* a) {
  const size_t n = static_cast<size_t>(a->num_replicas) * a->num_partitions;
  if (n > a->default_assignment_size) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "assignment buffer too small");
  for (size_t i = 0; i < n; ++i) a->default_assignment[i] = 0;
  return nullptr;
}

PJRT_Error* DeviceDescription_Id(PJRT_DeviceDescription_Id_Args* a) { a->id = 0; return nullptr; }
PJRT_Error* DeviceDescription_ProcessIndex(PJRT_DeviceDescription_ProcessIndex_Args* a) { a->process_index = 0; return nullptr; }
PJRT_Error* DeviceDescription_Attributes(PJRT_DeviceDescription_Attributes_Args* a) {
  a->num_attributes = 0;
  a->attributes = nullptr;
  return nullptr;
}
PJRT_Error* DeviceDescription_Kind(PJRT_DeviceDescription_Kind_Args* a) {
  a->device_kind = g_device_kind.c_str();
  a->device_kind_size = g_device_kind.size();
  return nullptr;
}
const char kDeviceString[] = "QmmB200Device(id=0)";
PJRT_Error* DeviceDescription_DebugString(PJRT_DeviceDescription_DebugString_Args* a) {
  a->debug_string = kDeviceString;
  a->debug_string_size = sizeof(kDeviceString) - 1;
  return nullptr;
}
PJRT_Error* DeviceDescription_ToString(PJRT_DeviceDescription_ToString_Args* a) {
  a->to_string = kDeviceString;
  a->to_string_size = sizeof(kDeviceString) - 1;
  return nullptr;
}
PJRT_Error* Device_GetDescription(PJRT_Device_GetDescription_Args* a) { a->device_description = &g_desc; return nullptr; }
PJRT_Error* Device_IsAddressable(PJRT_Device_IsAddressable_Args* a) { a->is_addressable = true; return nullptr; }
PJRT_Error* Device_LocalHardwareId(PJRT_Device_LocalHardwareId_Args* a) { a->local_hardware_id = 0; return nullptr; }
PJRT_Error* Device_AddressableMemories(PJRT_Device_AddressableMemories_Args* a) {
  a->memories = g_memories;
  a->num_memories = 1;
  return nullptr;
}
PJRT_Error* Device_DefaultMemory(PJRT_Device_DefaultMemory_Args* a) { a->memory = &g_memory; return nullptr; }

PJRT_Error* Memory_Id(PJRT_Memory_Id_Args* a) { a->id = 0; return nullptr; }
PJRT_Error* Memory_Kind(PJRT_Memory_Kind_Args* a) { a->kind = kMemoryKind; a->kind_size = sizeof(kMemoryKind) - 1; return nullptr; }
PJRT_Error* Memory_Kind_Id(PJRT_Memory_Kind_Id_Args* a) { a->kind_id = 0; return nullptr; }
const char kMemoryString[] = "QmmB200Memory(id=0, kind=device)";
PJRT_Error* Memory_DebugString(PJRT_Memory_DebugString_Args* a) {
  a->debug_string = kMemoryString;
  a->debug_string_size = sizeof(kMemoryString) - 1;
  return nullptr;
}
PJRT_Error* Memory_ToString(PJRT_Memory_ToString_Args* a) {
  a->to_string = kMemoryString;
  a->to_string_size = sizeof(kMemoryString) - 1;
  return nullptr;
}
PJRT_Error* Memory_AddressableByDevices(PJRT_Memory_AddressableByDevices_Args* a) {
  a->devices = g_devices;
  a->num_devices = 1;
  return nullptr;
}

// ---------------------------------------------------------------- compile

PJRT_Error* Client_Compile(PJRT_Client_Compile_Args* a) {
  if (PJRT_Error* e = EnsureEngine()) return e;
  if (!a->program || !a->program->code) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "no program");
  Gil gil;
  PyObject* code = PyBytes_FromStringAndSize(a->program->code, static_cast<Py_ssize_t>(a->program->code_size));
  PyObject* fmt = PyUnicode_FromStringAndSize(a->program->format, static_cast<Py_ssize_t>(a->program->format_size));
  PyObject* opts = a->compile_options
                       ? PyBytes_FromStringAndSize(a->compile_options, static_cast<Py_ssize_t>(a->compile_options_size))
                       : (Py_INCREF(Py_None), Py_None);
  PyObject* prog = (code && fmt && opts) ? PyObject_CallMethod(g_engine, "compile_program", "OOO", code, fmt, opts) : nullptr;
  Py_XDECREF(code); Py_XDECREF(fmt); Py_XDECREF(opts);
  if (!prog) return PyErrToErr("compile_program");
  auto* ex = new PJRT_Executable;
  ex->program = prog;
  std::vector<int64_t> types, nouts;
  bool ok = ReadString(prog, "name", &ex->name) && ReadString(prog, "fingerprint", &ex->fingerprint) &&
            ReadIntList(prog, "out_types", &types) && ReadIntList(prog, "donated_params", &ex->donated);
  PyObject* dims = ok ? PyObject_GetAttrString(prog, "out_dims") : nullptr;
  if (dims) {
    const Py_ssize_t n = PySequence_Size(dims);
    for (Py_ssize_t i = 0; i < n; ++i) {
      PyObject* d = PySequence_GetItem(dims, i);
      const Py_ssize_t r = d ? PySequence_Size(d) : 0;
      ex->dim_sizes.push_back(static_cast<size_t>(r));
      for (Py_ssize_t j = 0; j < r; ++j) {
        PyObject* it = PySequence_GetItem(d, j);
        ex->flat_dims.push_back(PyLong_AsLongLong(it));
        Py_XDECREF(it);
      }
      Py_XDECREF(d);
    }
    Py_DECREF(dims);
  }
  if (!ok || !dims || PyErr_Occurred()) {
    PJRT_Error* e = PyErrToErr("compile_program (metadata)");
    Py_DECREF(prog);
    delete ex;
    return e;
  }
  for (int64_t t : types) ex->out_types.push_back(static_cast<PJRT_Buffer_Type>(t));
  ex->num_outputs = ex->out_types.size();
  ex->memory_kinds.assign(ex->num_outputs, kMemoryKind);
  ex->memory_kind_sizes.assign(ex->num_outputs, sizeof(kMemoryKind) - 1);
  auto* le = new PJRT_LoadedExecutable;
  le->exec = ex;
  a->executable = le;
  return nullptr;
}

void ReleaseExecutable(PJRT_Executable* ex) {
  if (ex && --ex->refs == 0) {
    Gil gil;
    Py_XDECREF(ex->program);
    delete ex;
  }
}

PJRT_Error* Executable_Destroy(PJRT_Executable_Destroy_Args* a) { ReleaseExecutable(a->executable); return nullptr; }
PJRT_Error* Executable_Name(PJRT_Executable_Name_Args* a) {
  a->executable_name = a->executable->name.c_str();
  a->executable_name_size = a->executable->name.size();
  return nullptr;
}
PJRT_Error* Executable_NumReplicas(PJRT_Executable_NumReplicas_Args* a) { a->num_replicas = 1; return nullptr; }
PJRT_Error* Executable_NumPartitions(PJRT_Executable_NumPartitions_Args* a) { a->num_partitions = 1; return nullptr; }
PJRT_Error* Executable_NumOutputs(PJRT_Executable_NumOutputs_Args* a) { a->num_outputs = a->executable->num_outputs; return nullptr; }
PJRT_Error* Executable_SizeOfGeneratedCodeInBytes(PJRT_Executable_SizeOfGeneratedCodeInBytes_Args* a) {
  a->size_in_bytes = 0;    // nothing is generated: the program is interpreted
  return nullptr;
}
PJRT_Error* Executable_OutputMemoryKinds(PJRT_Executable_OutputMemoryKinds_Args* a) {
  a->num_outputs = a->executable->num_outputs;
  a->memory_kinds = a->executable->memory_kinds.data();
  a->memory_kind_sizes = a->executable->memory_kind_sizes.data();
  return nullptr;
}
PJRT_Error* Executable_OutputElementTypes(PJRT_Executable_OutputElementTypes_Args* a) {
  a->output_types = a->executable->out_types.data();
  a->num_output_types = a->executable->out_types.size();
  return nullptr;
}
PJRT_Error* Executable_OutputDimensions(PJRT_Executable_OutputDimensions_Args* a) {
  a->num_outputs = a->executable->num_outputs;
  a->dims = a->executable->flat_dims.data();
  a->dim_sizes = a->executable->dim_sizes.data();
  return nullptr;
}
PJRT_Error* Executable_Fingerprint(PJRT_Executable_Fingerprint_Args* a) {
  a->executable_fingerprint = a->executable->fingerprint.c_str();
  a->executable_fingerprint_size = a->executable->fingerprint.size();
  return nullptr;
}

PJRT_Error* LoadedExecutable_Destroy(PJRT_LoadedExecutable_Destroy_Args* a) {
  if (a->executable) {
    ReleaseExecutable(a->executable->exec);
    delete a->executable;
  }
  return nullptr;
}
PJRT_Error* LoadedExecutable_GetExecutable(PJRT_LoadedExecutable_GetExecutable_Args* a) {
  a->executable = a->loaded_executable->exec;
  ++a->executable->refs;               // the caller destroys it separately
  return nullptr;
}
PJRT_Error* LoadedExecutable_AddressableDevices(PJRT_LoadedExecutable_AddressableDevices_Args* a) {
  a->addressable_devices = g_devices;
  a->num_addressable_devices = 1;
  return nullptr;
}
PJRT_Error* LoadedExecutable_Delete(PJRT_LoadedExecutable_Delete_Args* a) { a->executable->deleted = true; return nullptr; }
PJRT_Error* LoadedExecutable_IsDeleted(PJRT_LoadedExecutable_IsDeleted_Args* a) { a->is_deleted = a->executable->deleted; return nullptr; }
PJRT_Error* LoadedExecutable_Fingerprint(PJRT_LoadedExecutable_Fingerprint_Args* a) {
  a->executable_fingerprint = a->executable->exec->fingerprint.c_str();
  a->executable_fingerprint_size = a->executable->exec->fingerprint.size();
  return nullptr;
}

// ---------------------------------------------------------------- execute

PJRT_Error* LoadedExecutable_Execute(PJRT_LoadedExecutable_Execute_Args* a) {
  if (PJRT_Error* e = EnsureEngine()) return e;
  if (a->num_devices != 1) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "there is one device");
  if (a->executable->deleted) return MakeError(PJRT_Error_Code_FAILED_PRECONDITION, "executable was deleted");
  PJRT_Executable* ex = a->executable->exec;
  Gil gil;
  PyObject* args = PyList_New(static_cast<Py_ssize_t>(a->num_args));
  if (!args) return PyErrToErr("execute");
  for (size_t i = 0; i < a->num_args; ++i) {
    PJRT_Buffer* b = a->argument_lists[0][i];
    if (!b || b->deleted || !b->py) {
      Py_DECREF(args);
      return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "argument " + std::to_string(i) + " is a deleted buffer");
    }
    Py_INCREF(b->py);
    PyList_SET_ITEM(args, static_cast<Py_ssize_t>(i), b->py);
  }
  PyObject* outs = PyObject_CallMethod(g_engine, "execute", "OO", ex->program, args);
  Py_DECREF(args);
  if (!outs) return PyErrToErr("execute");
  const Py_ssize_t n = PySequence_Size(outs);
  if (n != static_cast<Py_ssize_t>(ex->num_outputs)) {
    Py_DECREF(outs);
    return MakeError(PJRT_Error_Code_INTERNAL, "execute returned a different number of results than compile announced");
  }
  for (Py_ssize_t i = 0; i < n; ++i) a->output_lists[0][i] = WrapBuffer(PySequence_GetItem(outs, i));
  Py_DECREF(outs);
  // donated inputs are gone after the call (plugin/metal_pjrt.cc:1016-1038)
  for (int64_t d : ex->donated) {
    if (d < 0 || static_cast<size_t>(d) >= a->num_args) continue;
    bool keep = false;
    if (a->options)
      for (size_t k = 0; k < a->options->num_non_donatable_input_indices; ++k)
        keep = keep || a->options->non_donatable_input_indices[k] == d;
    PJRT_Buffer* b = a->argument_lists[0][d];
    if (!keep && b && !b->deleted) {
      Py_CLEAR(b->py);
      b->deleted = true;
    }
  }
  if (a->device_complete_events) a->device_complete_events[0] = ReadyEvent();
  return nullptr;
}

// ---------------------------------------------------------------- buffers

PJRT_Error* Client_BufferFromHostBuffer(PJRT_Client_BufferFromHostBuffer_Args* a) {
  if (PJRT_Error* e = EnsureEngine()) return e;
  // the byte range the strides reach (they may be negative: `data` can point inside the buffer)
  int64_t esize = 1;
  switch (a->type) {
    case PJRT_Buffer_Type_S16: case PJRT_Buffer_Type_U16: case PJRT_Buffer_Type_F16: case PJRT_Buffer_Type_BF16: esize = 2; break;
    case PJRT_Buffer_Type_S32: case PJRT_Buffer_Type_U32: case PJRT_Buffer_Type_F32: esize = 4; break;
    case PJRT_Buffer_Type_S64: case PJRT_Buffer_Type_U64: case PJRT_Buffer_Type_F64: case PJRT_Buffer_Type_C64: esize = 8; break;
    case PJRT_Buffer_Type_C128: esize = 16; break;
    default: esize = 1;
  }
  int64_t lo = 0, hi = esize, numel = 1;
  for (size_t d = 0; d < a->num_dims; ++d) numel *= a->dims[d];
  if (a->num_byte_strides) {
    if (a->num_byte_strides != a->num_dims) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "byte_strides and dims differ in length");
    for (size_t d = 0; d < a->num_dims; ++d) {
      const int64_t span = (a->dims[d] - 1) * a->byte_strides[d];
      if (a->dims[d] > 0) (span < 0 ? lo : hi) += span;
    }
  } else {
    hi = numel * esize;
  }
  Gil gil;
  PyObject* view = (a->data && numel > 0)
                       ? PyMemoryView_FromMemory(const_cast<char*>(static_cast<const char*>(a->data)) + lo, hi - lo, PyBUF_READ)
                       : (Py_INCREF(Py_None), Py_None);
  PyObject* dims = PyTuple_New(static_cast<Py_ssize_t>(a->num_dims));
  for (size_t d = 0; d < a->num_dims; ++d) PyTuple_SET_ITEM(dims, static_cast<Py_ssize_t>(d), PyLong_FromLongLong(a->dims[d]));
  PyObject* strides;
  if (a->num_byte_strides) {
    strides = PyTuple_New(static_cast<Py_ssize_t>(a->num_dims));
    for (size_t d = 0; d < a->num_dims; ++d) PyTuple_SET_ITEM(strides, static_cast<Py_ssize_t>(d), PyLong_FromLongLong(a->byte_strides[d]));
  } else {
    strides = (Py_INCREF(Py_None), Py_None);
  }
  PyObject* buf = (view && dims && strides)
                      ? PyObject_CallMethod(g_engine, "buffer_from_host", "OiOOL", view, static_cast<int>(a->type), dims, strides,
                                            static_cast<long long>(-lo))
                      : nullptr;
  Py_XDECREF(view); Py_XDECREF(dims); Py_XDECREF(strides);
  if (!buf) return PyErrToErr("buffer_from_host");
  a->buffer = WrapBuffer(buf);
  a->done_with_host_buffer = ReadyEvent();      // the bytes were copied before returning
  return nullptr;
}

PJRT_Error* Buffer_Destroy(PJRT_Buffer_Destroy_Args* a) {
  if (a->buffer) {
    if (a->buffer->py) {
      Gil gil;
      Py_CLEAR(a->buffer->py);
    }
    delete a->buffer;
  }
  return nullptr;
}
PJRT_Error* Buffer_ElementType(PJRT_Buffer_ElementType_Args* a) { a->type = a->buffer->type; return nullptr; }
PJRT_Error* Buffer_Dimensions(PJRT_Buffer_Dimensions_Args* a) {
  a->dims = a->buffer->dims.data();
  a->num_dims = a->buffer->dims.size();
  return nullptr;
}
PJRT_Error* Buffer_UnpaddedDimensions(PJRT_Buffer_UnpaddedDimensions_Args* a) {
  a->unpadded_dims = a->buffer->dims.data();
  a->num_dims = a->buffer->dims.size();
  return nullptr;
}
PJRT_Error* Buffer_DynamicDimensionIndices(PJRT_Buffer_DynamicDimensionIndices_Args* a) {
  a->dynamic_dim_indices = nullptr;
  a->num_dynamic_dims = 0;
  return nullptr;
}
PJRT_Error* Buffer_OnDeviceSizeInBytes(PJRT_Buffer_OnDeviceSizeInBytes_Args* a) { a->on_device_size_in_bytes = a->buffer->nbytes; return nullptr; }
PJRT_Error* Buffer_Device(PJRT_Buffer_Device_Args* a) { a->device = &g_device; return nullptr; }
PJRT_Error* Buffer_Memory(PJRT_Buffer_Memory_Args* a) { a->memory = &g_memory; return nullptr; }
PJRT_Error* Buffer_Delete(PJRT_Buffer_Delete_Args* a) {
  if (a->buffer->py) {
    Gil gil;
    Py_CLEAR(a->buffer->py);
  }
  a->buffer->deleted = true;
  return nullptr;
}
PJRT_Error* Buffer_IsDeleted(PJRT_Buffer_IsDeleted_Args* a) { a->is_deleted = a->buffer->deleted; return nullptr; }
PJRT_Error* Buffer_IsOnCpu(PJRT_Buffer_IsOnCpu_Args* a) { a->is_on_cpu = false; return nullptr; }
PJRT_Error* Buffer_ReadyEvent(PJRT_Buffer_ReadyEvent_Args* a) { a->event = ReadyEvent(); return nullptr; }
PJRT_Error* Buffer_CopyToDevice(PJRT_Buffer_CopyToDevice_Args* a) {
  if (a->buffer->deleted) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "buffer was deleted");
  Gil gil;                                         // one device: a second handle on the same array
  auto* b = new PJRT_Buffer(*a->buffer);
  Py_XINCREF(b->py);
  a->dst_buffer = b;
  return nullptr;
}
PJRT_Error* Buffer_ToHostBuffer(PJRT_Buffer_ToHostBuffer_Args* a) {
  if (a->src->deleted || !a->src->py) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "buffer was deleted");
  if (!a->dst) {                                   // size query
    a->dst_size = a->src->nbytes;
    a->event = nullptr;
    return nullptr;
  }
  if (a->dst_size < a->src->nbytes) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "destination too small");
  Gil gil;
  PyObject* bytes = PyObject_CallMethod(g_engine, "to_host", "O", a->src->py);
  if (!bytes) return PyErrToErr("to_host");
  char* ptr = nullptr;
  Py_ssize_t n = 0;
  if (PyBytes_AsStringAndSize(bytes, &ptr, &n) != 0 || static_cast<size_t>(n) != a->src->nbytes) {
    Py_DECREF(bytes);
    PyErr_Clear();
    return MakeError(PJRT_Error_Code_INTERNAL, "to_host returned a different number of bytes");
  }
  memcpy(a->dst, ptr, static_cast<size_t>(n));
  Py_DECREF(bytes);
  a->event = ReadyEvent();
  return nullptr;
}
PJRT_Error* Buffer_UnsafePointer(PJRT_Buffer_UnsafePointer_Args* a) {
  if (a->buffer->deleted || !a->buffer->py) return MakeError(PJRT_Error_Code_INVALID_ARGUMENT, "buffer was deleted");
  Gil gil;
  PyObject* p = PyObject_CallMethod(g_engine, "buffer_pointer", "O", a->buffer->py);
  if (!p) return PyErrToErr("buffer_pointer");
  a->buffer_pointer = static_cast<uintptr_t>(PyLong_AsUnsignedLongLong(p));
  Py_DECREF(p);
  return nullptr;
}

// ---------------------------------------------------------------- the table

// A named UNIMPLEMENTED stub for every entry of PJRT_Api (the list of entries is generated
// from the header at build time), then the implemented ones on top.
#define X(name) \
  PJRT_Error* name##_Unimplemented(void*) { return MakeError(PJRT_Error_Code_UNIMPLEMENTED, #name " is not implemented by the qmm_b200 plugin"); }
#include "pjrt_api_fields.inc"
#undef X

PJRT_Api g_api;
std::once_flag g_api_once;

void BuildApi() {
  memset(&g_api, 0, sizeof(g_api));
  g_api.struct_size = PJRT_Api_STRUCT_SIZE;
  g_api.extension_start = nullptr;
  g_api.pjrt_api_version.struct_size = PJRT_Api_Version_STRUCT_SIZE;
  g_api.pjrt_api_version.extension_start = nullptr;
  g_api.pjrt_api_version.major_version = PJRT_API_MAJOR;
  g_api.pjrt_api_version.minor_version = PJRT_API_MINOR;
#define X(name) g_api.name = reinterpret_cast<name*>(&name##_Unimplemented);
#include "pjrt_api_fields.inc"
#undef X
#define SET(name) g_api.PJRT_##name = name
  SET(Error_Destroy); SET(Error_Message); SET(Error_GetCode);
  SET(Plugin_Initialize); SET(Plugin_Attributes);
  SET(Event_Destroy); SET(Event_IsReady); SET(Event_Error); SET(Event_Await); SET(Event_OnReady);
  SET(Client_Create); SET(Client_Destroy); SET(Client_PlatformName); SET(Client_ProcessIndex); SET(Client_PlatformVersion);
  SET(Client_Devices); SET(Client_AddressableDevices); SET(Client_LookupDevice); SET(Client_LookupAddressableDevice);
  SET(Client_AddressableMemories); SET(Client_Compile); SET(Client_DefaultDeviceAssignment); SET(Client_BufferFromHostBuffer);
  SET(DeviceDescription_Id); SET(DeviceDescription_ProcessIndex); SET(DeviceDescription_Attributes);
  SET(DeviceDescription_Kind); SET(DeviceDescription_DebugString); SET(DeviceDescription_ToString);
  SET(Device_GetDescription); SET(Device_IsAddressable); SET(Device_LocalHardwareId); SET(Device_AddressableMemories);
  SET(Device_DefaultMemory);
  SET(Memory_Id); SET(Memory_Kind); SET(Memory_Kind_Id); SET(Memory_DebugString); SET(Memory_ToString); SET(Memory_AddressableByDevices);
  SET(Executable_Destroy); SET(Executable_Name); SET(Executable_NumReplicas); SET(Executable_NumPartitions);
  SET(Executable_NumOutputs); SET(Executable_SizeOfGeneratedCodeInBytes); SET(Executable_OutputMemoryKinds);
  SET(Executable_OutputElementTypes); SET(Executable_OutputDimensions); SET(Executable_Fingerprint);
  SET(LoadedExecutable_Destroy); SET(LoadedExecutable_GetExecutable); SET(LoadedExecutable_AddressableDevices);
  SET(LoadedExecutable_Delete); SET(LoadedExecutable_IsDeleted); SET(LoadedExecutable_Execute); SET(LoadedExecutable_Fingerprint);
  SET(Buffer_Destroy); SET(Buffer_ElementType); SET(Buffer_Dimensions); SET(Buffer_UnpaddedDimensions);
  SET(Buffer_DynamicDimensionIndices); SET(Buffer_OnDeviceSizeInBytes); SET(Buffer_Device); SET(Buffer_Memory);
  SET(Buffer_Delete); SET(Buffer_IsDeleted); SET(Buffer_CopyToDevice); SET(Buffer_ToHostBuffer); SET(Buffer_IsOnCpu);
  SET(Buffer_ReadyEvent); SET(Buffer_UnsafePointer);
#undef SET
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const PJRT_Api* GetPjrtApi() {
  std::call_once(g_api_once, BuildApi);
  return &g_api;
}
