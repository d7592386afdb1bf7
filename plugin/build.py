"""Builds the PJRT entry (`libqmm_pjrt.so`) and its C++ test host (`pjrt_driver`) in-tree.

    python plugin/build.py [--force]

Both compile against openxla's `pjrt_c_api.h` (PJRT C API 0.114, the version the reference
vendors under plugin/vendor/). The header is not part of this repository: its directory is taken
from $PJRT_C_API_INCLUDE, else from a checkout of the reference next to this repository
(`../reference/plugin/vendor`). Without it the build is skipped (the built files travel with the
tree) and `build()` returns None. The list of `PJRT_Api` entries is read from the header itself,
so that every entry outside the implemented subset gets its own UNIMPLEMENTED stub.
"""

from __future__ import annotations

import os
import re
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
PLUGIN = os.path.join(HERE, "libqmm_pjrt.so")
DRIVER = os.path.join(HERE, "pjrt_driver")


def header_dir():
    cands = [os.environ.get("PJRT_C_API_INCLUDE"), os.path.join(HERE, "..", "..", "reference", "plugin", "vendor")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "pjrt_c_api.h")):
            return os.path.abspath(c)
    return None


def api_fields(header: str) -> list[str]:
    text = open(header).read()
    body = text[text.index("typedef struct PJRT_Api {"):text.index("} PJRT_Api;")]
    return re.findall(r"_PJRT_API_STRUCT_FIELD\(\s*(PJRT_\w+)\s*\)", body)


def stale(out, deps):
    return not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps)


def build(force: bool = False):
    inc = header_dir()
    if inc is None:
        return None
    gen = os.path.join(HERE, "build")
    os.makedirs(gen, exist_ok=True)
    fields = api_fields(os.path.join(inc, "pjrt_c_api.h"))
    with open(os.path.join(gen, "pjrt_api_fields.inc"), "w") as f:
        f.write("".join(f"X({name})\n" for name in fields))
    py_inc = sysconfig.get_config_var("INCLUDEPY")
    libdir = sysconfig.get_config_var("LIBDIR")
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    src, drv = os.path.join(HERE, "qmm_pjrt.cc"), os.path.join(HERE, "pjrt_driver.cc")
    if force or stale(PLUGIN, [src, __file__]):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=hidden", f"-I{inc}", f"-I{gen}",
                               f"-I{py_inc}", src, "-o", PLUGIN + ".tmp", f"-L{libdir}", f"-lpython{ver}", "-ldl", "-lpthread",
                               f"-Wl,-rpath,{libdir}"])
        os.replace(PLUGIN + ".tmp", PLUGIN)
    if force or stale(DRIVER, [drv, __file__]):
        subprocess.check_call(["g++", "-std=c++17", "-O2", f"-I{inc}", drv, "-o", DRIVER, "-ldl"])
    return PLUGIN


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
