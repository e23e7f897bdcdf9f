"""The C API driven from a separate C program (its own process: the library starts its own interpreter)."""
import os
import shutil
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "transformers_fusion_b200", "lib")

C_MAIN = r'''
#include <stdio.h>
#include <string.h>
#include "tfb_capi.h"
int main(int argc, char** argv) {
  quant_model* bad = quant_model_load("/nonexistent/model.quant");
  if (bad != NULL || strlen(quant_last_error()) == 0) { printf("FAIL: missing file accepted\n"); return 2; }
  printf("ERR=%s\n", quant_last_error());
  quant_model* m = quant_model_load(argv[1]);
  if (!m) { printf("FAIL load: %s\n", quant_last_error()); return 3; }
  char* a = quant_generate(m, "hello", 8, 0.0f, 1, 1.0f);
  char* b = quant_generate(m, "hello", 8, 0.0f, 1, 1.0f);
  if (!a || !b) { printf("FAIL gen: %s\n", quant_last_error()); return 4; }
  printf("SAME=%d LEN=%d\n", strcmp(a, b) == 0, (int)strlen(a));
  quant_free_string(a); quant_free_string(b);
  quant_model_free(m);
  return 0;
}
'''


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs a C compiler")
def test_c_program_loads_and_generates(tmp_path):
    from transformers_fusion_b200 import build
    so = build.build_capi()
    if so is None:
        pytest.skip("Python development headers are not installed")
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.quant import codec
    m = DenseModel(TransformerConfig(vocab_size=259, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=64),
                   device="cpu", dtype=torch.float32, seed=0)
    codec.save_model(m, tmp_path / "m.quant")
    (tmp_path / "main.c").write_text(C_MAIN)
    exe = tmp_path / "main"
    inc = os.path.join(ROOT, "transformers_fusion_b200", "csrc", "capi")
    subprocess.run(["gcc", str(tmp_path / "main.c"), "-I", inc, f"-L{LIB}", "-ltfb_capi", f"-Wl,-rpath,{LIB}", "-o", str(exe)], check=True)
    site = [p for p in sys.path if p.endswith("site-packages")]
    env = dict(os.environ, TFB_PYTHONPATH=ROOT, PYTHONPATH=os.pathsep.join([ROOT] + site), CUDA_VISIBLE_DEVICES="", TFB_DEVICE="cpu")
    r = subprocess.run([str(exe), str(tmp_path / "m.quant")], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ERR=load failed" in r.stdout and "SAME=1" in r.stdout
