"""The C header of the kernels: a C program that includes ``photon/kernels.h``, takes the address of every
declared entry point and calls one of them links against the built libraries and runs (on the CPU: the call is
the host-only ``photon_static_error_string``).  The kernel sources include the same header, so their definitions
already had to match it to compile."""
import os
import re
import shutil
import subprocess

import pytest

from photon_infer_b200.csrc.build import ALL_MODULES, INCLUDE_DIR, compile_module, find_nvcc

HEADER = os.path.join(INCLUDE_DIR, "photon", "kernels.h")


def _declared():
    text = open(HEADER).read()
    return re.findall(r"^PHOTON_EXPORT\s+(?:int|const char\*)\s+(photon_\w+)\(", text, flags=re.M)


def test_header_declares_every_exported_entry_point():
    """What the sources export (PHOTON_API) is what the header declares, no more and no less."""
    src_dir = os.path.dirname(INCLUDE_DIR) + "/csrc"
    exported = set()
    for name in os.listdir(src_dir):
        if name.endswith(".cu"):
            body = open(os.path.join(src_dir, name)).read()
            body = re.sub(r"#ifdef AD_TRACE.*?#else", "", body, flags=re.S)     # a debug build's extra symbol
            exported.update(re.findall(r"PHOTON_API\s+(?:int|const char\*)\s+(photon_\w+)\(", body))
    assert exported == set(_declared())


def test_c_program_links_against_the_libraries(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    cuda_home = os.path.dirname(os.path.dirname(find_nvcc()))
    libs = [compile_module(m) for m in ALL_MODULES]
    libs += [compile_module(m, {"HEAD_DIM": 64}) for m in ("attention_flash", "attention_tc", "attention_decode")]
    names = _declared()
    src = tmp_path / "use_header.c"
    src.write_text(
        "#include <stdio.h>\n#include <string.h>\n#include <photon/kernels.h>\n"
        "int main(void) {\n  const void* entry[] = {" + ", ".join(f"(const void*){n}" for n in names) + "};\n"
        "  for (unsigned i = 0; i < sizeof(entry) / sizeof(entry[0]); ++i) if (entry[i] == 0) return 2;\n"
        "  const char* words = photon_static_error_string(PHOTON_ERR_UNSUPPORTED);\n"
        "  printf(\"%u entry points; -2 means: %s\\n\", (unsigned)(sizeof(entry) / sizeof(entry[0])), words);\n"
        "  return strstr(words, \"multiples of 8\") ? 0 : 3;\n}\n")
    exe = tmp_path / "use_header"
    cmd = [cc, "-std=c11", "-Wall", "-Werror", "-I", INCLUDE_DIR, "-I", os.path.join(cuda_home, "include"), str(src),
           "-o", str(exe), *libs, f"-L{cuda_home}/lib64", "-lcudart", "-lstdc++",
           "-Wl,-rpath," + os.path.dirname(libs[0]), f"-Wl,-rpath,{cuda_home}/lib64"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert f"{len(names)} entry points" in run.stdout
