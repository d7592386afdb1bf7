// A PJRT host in C++ for tests: loads the plugin the way jaxlib does (dlopen + GetPjrtApi),
// compiles a StableHLO text program, moves host arrays in, executes, moves results out.
//
//   pjrt_driver <plugin.so> <program.mlir> <out_prefix> [<file>:<PJRT_Buffer_Type>:<d0>x<d1>...]...
//
// Results go to <out_prefix>.<i>.bin (out_prefix "-": stop after compiling, no device needed); what the client reports goes to stdout as `key=value` lines.
// Also exercises the error paths: a bytecode artifact and an unknown format must be refused
// with UNIMPLEMENTED, a malformed program with an error, an entry outside the implemented
// subset with UNIMPLEMENTED, and a call with a wrong argument count with INVALID_ARGUMENT.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "pjrt_c_api.h"

static const PJRT_Api* api = nullptr;

static std::string ErrText(PJRT_Error* e, int* code = nullptr) {
  if (!e) return "";
  PJRT_Error_Message_Args m = {};
  m.struct_size = PJRT_Error_Message_Args_STRUCT_SIZE;
  m.error = e;
  api->PJRT_Error_Message(&m);
  PJRT_Error_GetCode_Args c = {};
  c.struct_size = PJRT_Error_GetCode_Args_STRUCT_SIZE;
  c.error = e;
  api->PJRT_Error_GetCode(&c);
  if (code) *code = static_cast<int>(c.code);
  std::string s(m.message, m.message_size);
  PJRT_Error_Destroy_Args d = {};
  d.struct_size = PJRT_Error_Destroy_Args_STRUCT_SIZE;
  d.error = e;
  api->PJRT_Error_Destroy(&d);
  return s;
}

#define CHECK_OK(expr)                                                   \
  do {                                                                   \
    PJRT_Error* _e = (expr);                                             \
    if (_e) {                                                            \
      printf("FAILED %s: %s\n", #expr, ErrText(_e).c_str());             \
      return 1;                                                          \
    }                                                                    \
  } while (0)

static std::string ReadFile(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static PJRT_Error* Compile(PJRT_Client* client, const std::string& code, const char* fmt, PJRT_LoadedExecutable** out) {
  PJRT_Program prog = {};
  prog.struct_size = PJRT_Program_STRUCT_SIZE;
  prog.code = const_cast<char*>(code.data());
  prog.code_size = code.size();
  prog.format = fmt;
  prog.format_size = strlen(fmt);
  PJRT_Client_Compile_Args a = {};
  a.struct_size = PJRT_Client_Compile_Args_STRUCT_SIZE;
  a.client = client;
  a.program = &prog;
  PJRT_Error* e = api->PJRT_Client_Compile(&a);
  *out = a.executable;
  return e;
}

int main(int argc, char** argv) {
  if (argc < 4) {
    fprintf(stderr, "usage: pjrt_driver plugin.so program.mlir out_prefix [file:type:dims]...\n");
    return 2;
  }
  void* h = dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    printf("FAILED dlopen: %s\n", dlerror());
    return 1;
  }
  auto get = reinterpret_cast<const PJRT_Api* (*)()>(dlsym(h, "GetPjrtApi"));
  if (!get) {
    printf("FAILED no GetPjrtApi\n");
    return 1;
  }
  api = get();
  printf("api_version=%d.%d\n", api->pjrt_api_version.major_version, api->pjrt_api_version.minor_version);

  PJRT_Plugin_Initialize_Args init = {};
  init.struct_size = PJRT_Plugin_Initialize_Args_STRUCT_SIZE;
  CHECK_OK(api->PJRT_Plugin_Initialize(&init));
  PJRT_Client_Create_Args cc = {};
  cc.struct_size = PJRT_Client_Create_Args_STRUCT_SIZE;
  CHECK_OK(api->PJRT_Client_Create(&cc));
  PJRT_Client* client = cc.client;

  PJRT_Client_PlatformName_Args pn = {};
  pn.struct_size = PJRT_Client_PlatformName_Args_STRUCT_SIZE;
  pn.client = client;
  CHECK_OK(api->PJRT_Client_PlatformName(&pn));
  printf("platform=%.*s\n", static_cast<int>(pn.platform_name_size), pn.platform_name);
  PJRT_Client_AddressableDevices_Args ad = {};
  ad.struct_size = PJRT_Client_AddressableDevices_Args_STRUCT_SIZE;
  ad.client = client;
  CHECK_OK(api->PJRT_Client_AddressableDevices(&ad));
  printf("devices=%zu\n", ad.num_addressable_devices);
  PJRT_Device_GetDescription_Args gd = {};
  gd.struct_size = PJRT_Device_GetDescription_Args_STRUCT_SIZE;
  gd.device = ad.addressable_devices[0];
  CHECK_OK(api->PJRT_Device_GetDescription(&gd));
  PJRT_DeviceDescription_Kind_Args dk = {};
  dk.struct_size = PJRT_DeviceDescription_Kind_Args_STRUCT_SIZE;
  dk.device_description = gd.device_description;
  CHECK_OK(api->PJRT_DeviceDescription_Kind(&dk));
  printf("device_kind=%.*s\n", static_cast<int>(dk.device_kind_size), dk.device_kind);

  // ---- error paths ----
  int code = 0;
  PJRT_LoadedExecutable* bad = nullptr;
  std::string msg = ErrText(Compile(client, std::string("ML\xefR\x01junk", 9), "mlir", &bad), &code);
  printf("bytecode_code=%d\n", code);
  msg = ErrText(Compile(client, "module {}", "hlo", &bad), &code);
  printf("format_code=%d\n", code);
  msg = ErrText(Compile(client, "this is not a program", "mlir", &bad), &code);
  printf("garbage_code=%d\n", code);
  PJRT_Client_TopologyDescription_Args td = {};
  td.struct_size = PJRT_Client_TopologyDescription_Args_STRUCT_SIZE;
  td.client = client;
  msg = ErrText(api->PJRT_Client_TopologyDescription(&td), &code);
  printf("topology_code=%d message=%s\n", code, msg.c_str());

  // ---- the program ----
  PJRT_LoadedExecutable* exe = nullptr;
  CHECK_OK(Compile(client, ReadFile(argv[2]), "mlir", &exe));
  PJRT_LoadedExecutable_GetExecutable_Args ge = {};
  ge.struct_size = PJRT_LoadedExecutable_GetExecutable_Args_STRUCT_SIZE;
  ge.loaded_executable = exe;
  CHECK_OK(api->PJRT_LoadedExecutable_GetExecutable(&ge));
  PJRT_Executable_Name_Args en = {};
  en.struct_size = PJRT_Executable_Name_Args_STRUCT_SIZE;
  en.executable = ge.executable;
  CHECK_OK(api->PJRT_Executable_Name(&en));
  printf("name=%.*s\n", static_cast<int>(en.executable_name_size), en.executable_name);
  PJRT_Executable_NumOutputs_Args no = {};
  no.struct_size = PJRT_Executable_NumOutputs_Args_STRUCT_SIZE;
  no.executable = ge.executable;
  CHECK_OK(api->PJRT_Executable_NumOutputs(&no));
  printf("num_outputs=%zu\n", no.num_outputs);
  PJRT_Executable_OutputDimensions_Args od = {};
  od.struct_size = PJRT_Executable_OutputDimensions_Args_STRUCT_SIZE;
  od.executable = ge.executable;
  CHECK_OK(api->PJRT_Executable_OutputDimensions(&od));
  PJRT_Executable_OutputElementTypes_Args ot = {};
  ot.struct_size = PJRT_Executable_OutputElementTypes_Args_STRUCT_SIZE;
  ot.executable = ge.executable;
  CHECK_OK(api->PJRT_Executable_OutputElementTypes(&ot));
  size_t at = 0;
  for (size_t i = 0; i < od.num_outputs; ++i) {
    printf("output%zu=type %d dims", i, static_cast<int>(ot.output_types[i]));
    for (size_t j = 0; j < od.dim_sizes[i]; ++j) printf(" %lld", static_cast<long long>(od.dims[at++]));
    printf("\n");
  }

  if (std::string(argv[3]) == "-") {      // metadata only (no device needed)
    printf("done=1\n");
    return 0;
  }

  // ---- arguments ----
  std::vector<PJRT_Buffer*> bufs;
  std::vector<std::string> blobs;
  for (int i = 4; i < argc; ++i) {
    std::string spec = argv[i];
    const size_t c1 = spec.find(':'), c2 = spec.find(':', c1 + 1);
    blobs.push_back(ReadFile(spec.substr(0, c1)));
    const int type = atoi(spec.substr(c1 + 1, c2 - c1 - 1).c_str());
    std::vector<int64_t> dims;
    std::stringstream ds(spec.substr(c2 + 1));
    std::string tok;
    while (std::getline(ds, tok, 'x')) dims.push_back(atoll(tok.c_str()));
    PJRT_Client_BufferFromHostBuffer_Args bh = {};
    bh.struct_size = PJRT_Client_BufferFromHostBuffer_Args_STRUCT_SIZE;
    bh.client = client;
    bh.data = blobs.back().data();
    bh.type = static_cast<PJRT_Buffer_Type>(type);
    bh.dims = dims.data();
    bh.num_dims = dims.size();
    bh.host_buffer_semantics = PJRT_HostBufferSemantics_kImmutableOnlyDuringCall;
    bh.device = ad.addressable_devices[0];
    CHECK_OK(api->PJRT_Client_BufferFromHostBuffer(&bh));
    PJRT_Event_Destroy_Args ed = {};
    ed.struct_size = PJRT_Event_Destroy_Args_STRUCT_SIZE;
    ed.event = bh.done_with_host_buffer;
    CHECK_OK(api->PJRT_Event_Destroy(&ed));
    bufs.push_back(bh.buffer);
  }

  // ---- execute twice (the second call reuses the pack), plus one call with a missing argument ----
  std::vector<PJRT_Buffer*> outs(no.num_outputs, nullptr);
  for (int round = 0; round < 3; ++round) {
    PJRT_ExecuteOptions opts = {};
    opts.struct_size = PJRT_ExecuteOptions_STRUCT_SIZE;
    PJRT_Buffer* const* arg_list = bufs.data();
    PJRT_Buffer** out_list = outs.data();
    PJRT_Event* done = nullptr;
    PJRT_LoadedExecutable_Execute_Args ex = {};
    ex.struct_size = PJRT_LoadedExecutable_Execute_Args_STRUCT_SIZE;
    ex.executable = exe;
    ex.options = &opts;
    ex.argument_lists = &arg_list;
    ex.num_devices = 1;
    ex.num_args = round == 2 ? bufs.size() - 1 : bufs.size();
    ex.output_lists = &out_list;
    ex.device_complete_events = &done;
    PJRT_Error* e = api->PJRT_LoadedExecutable_Execute(&ex);
    if (round == 2) {
      ErrText(e, &code);
      printf("short_call_code=%d\n", e ? code : 0);
      break;
    }
    CHECK_OK(e);
    PJRT_Event_Destroy_Args ed = {};
    ed.struct_size = PJRT_Event_Destroy_Args_STRUCT_SIZE;
    ed.event = done;
    CHECK_OK(api->PJRT_Event_Destroy(&ed));
    for (size_t i = 0; i < outs.size(); ++i) {
      PJRT_Buffer_ToHostBuffer_Args th = {};
      th.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
      th.src = outs[i];
      CHECK_OK(api->PJRT_Buffer_ToHostBuffer(&th));          // size query
      std::vector<char> host(th.dst_size);
      th.dst = host.data();
      CHECK_OK(api->PJRT_Buffer_ToHostBuffer(&th));
      if (round == 1) {
        std::ofstream f(std::string(argv[3]) + "." + std::to_string(i) + ".bin", std::ios::binary);
        f.write(host.data(), static_cast<std::streamsize>(host.size()));
        printf("result%zu_bytes=%zu\n", i, host.size());
      }
      PJRT_Buffer_Destroy_Args bd = {};
      bd.struct_size = PJRT_Buffer_Destroy_Args_STRUCT_SIZE;
      bd.buffer = outs[i];
      CHECK_OK(api->PJRT_Buffer_Destroy(&bd));
    }
  }
  for (PJRT_Buffer* b : bufs) {
    PJRT_Buffer_Destroy_Args bd = {};
    bd.struct_size = PJRT_Buffer_Destroy_Args_STRUCT_SIZE;
    bd.buffer = b;
    CHECK_OK(api->PJRT_Buffer_Destroy(&bd));
  }
  PJRT_Executable_Destroy_Args xd = {};
  xd.struct_size = PJRT_Executable_Destroy_Args_STRUCT_SIZE;
  xd.executable = ge.executable;
  CHECK_OK(api->PJRT_Executable_Destroy(&xd));
  PJRT_LoadedExecutable_Destroy_Args ld = {};
  ld.struct_size = PJRT_LoadedExecutable_Destroy_Args_STRUCT_SIZE;
  ld.executable = exe;
  CHECK_OK(api->PJRT_LoadedExecutable_Destroy(&ld));
  printf("done=1\n");
  return 0;
}
