"""C API: in-process through ctypes (joins the running interpreter) and from a stand-alone C
program that embeds the interpreter."""
import ctypes
import os
import shutil
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "mythos_b200", "liboil_capi.so")

pytestmark = pytest.mark.skipif(not os.path.exists(LIB), reason="liboil_capi.so not built")


def _tiny_model(path):
    from mythos_b200.models import DenseModel
    from mythos_b200.models.config import tiny_byte_config
    from mythos_b200.oil.model_io import save_model

    torch.manual_seed(0)
    cfg = tiny_byte_config()
    cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden_size = 1, 64, 1, 128
    save_model(DenseModel(cfg), path)


def test_capi_in_process(tmp_path):
    path = str(tmp_path / "m.oil")
    _tiny_model(path)
    lib = ctypes.CDLL(LIB)
    lib.oil_model_load_on.restype = ctypes.c_void_p
    lib.oil_model_load_on.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.oil_generate.restype = ctypes.c_void_p
    lib.oil_generate.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    lib.oil_last_error.restype = ctypes.c_char_p
    lib.oil_free_string.argtypes = [ctypes.c_void_p]
    lib.oil_model_free.argtypes = [ctypes.c_void_p]
    assert lib.oil_model_load_on(b"/nonexistent/model.oil", b"cpu") is None
    assert b"nonexistent" in lib.oil_last_error()
    m = lib.oil_model_load_on(path.encode(), b"cpu")
    assert m, lib.oil_last_error()
    s = lib.oil_generate(m, b"ab", 5)
    assert s, lib.oil_last_error()
    a = ctypes.string_at(s)
    lib.oil_free_string(s)
    s2 = lib.oil_generate(m, b"ab", 5)
    assert ctypes.string_at(s2) == a        # greedy decoding is deterministic
    lib.oil_free_string(s2)
    lib.oil_model_free(m)
    assert lib.oil_generate_binding(b"java", b"/tmp") == 0 and b"not implemented" in lib.oil_last_error()


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_capi_from_c_program(tmp_path):
    path = str(tmp_path / "m.oil")
    _tiny_model(path)
    src = tmp_path / "main.c"
    src.write_text('''
#include <stdio.h>
#include "oil_c_api.h"
int main(int argc, char** argv) {
  OilModel* m = oil_model_load_on(argv[1], "cpu");
  if (!m) { fprintf(stderr, "load failed: %s\\n", oil_last_error()); return 1; }
  char* out = oil_generate(m, "hi", 4);
  if (!out) { fprintf(stderr, "generate failed: %s\\n", oil_last_error()); return 2; }
  printf("OK[%s]\\n", out);
  oil_free_string(out);
  oil_model_free(m);
  return 0;
}
''')
    exe = str(tmp_path / "main")
    inc = os.path.join(ROOT, "mythos_b200", "csrc", "capi")
    subprocess.run(["gcc", str(src), "-I", inc, "-L", os.path.dirname(LIB), "-loil_capi",
                    "-Wl,-rpath," + os.path.dirname(LIB), "-o", exe], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p),
               PYTHONHOME=sys.base_prefix)
    r = subprocess.run([exe, path], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("OK["), r.stderr[-2000:]
