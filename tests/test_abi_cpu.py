"""CPU-side checks of the boundary: the library loads without a GPU, exports every symbol
the header declares, and the parameter sets have the sizes the workloads name."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "optengine.h"), encoding="utf-8").read()
    return sorted(set(re.findall(r"^OE_API\s+[\w\s\*]+?\b(oe_\w+)\s*\(", text, flags=re.M)))


def test_header_symbols_are_exported_and_bound():
    from gograd_b200 import _lib
    handle = C.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(handle, name), f"{name} declared in optengine.h but not exported"
    assert sorted(_lib.PROTOTYPES) == names, "ctypes prototypes and header disagree"
    assert _lib.lib().oe_abi_version() == 1


def test_struct_layouts_match_the_header():
    from gograd_b200 import _lib
    assert C.sizeof(_lib.oe_tensor_desc) == 56
    assert C.sizeof(_lib.oe_adamw_hparams) == 48
    assert C.sizeof(_lib.oe_sgd_hparams) == 40
    assert _lib.oe_adamw_hparams.step_dev.offset == 32
    assert C.sizeof(_lib.oe_zero1_desc) == 320 and _lib.oe_zero1_desc.sync_blocks.offset == 160
    assert _lib.oe_zero1_desc.shadow_mc_delta.offset == 152 and _lib.oe_zero1_desc.timeout_ms.offset == 224


def test_no_cpu_fallback_without_a_driver():
    """On a machine without a CUDA driver every device call fails loudly with a message."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from gograd_b200 import _lib
    lib = _lib.lib()
    rc = lib.oe_init(0)
    assert rc == _lib.OE_ERR_NO_DRIVER and b"driver" in lib.oe_last_error().lower()
    out = C.c_void_p()
    desc = (_lib.oe_tensor_desc * 1)()
    assert lib.oe_plan_create(0, desc, 1, 0, C.byref(out)) != 0 and not out.value
    assert lib.oe_cast_bf16(0, 16, 16, 4, 0) != 0
    assert lib.oe_grad_norm_static(0, 16, 4, 16, 0) != 0
    with pytest.raises(_lib.EngineError):
        import gograd_b200
        gograd_b200.init(0)


def test_parameter_set_sizes():
    from gograd_b200 import paramsets
    for key, want in paramsets.EXPECTED_NUMEL.items():
        ps = paramsets.get(key)
        assert ps.numel == want, key
    assert [len(paramsets.get(k).params) for k in ("mlp", "cnn", "gpt", "llama1b", "llama8b")] == [4, 14, 145, 219, 291]
    sample = paramsets.scaled(paramsets.get("llama1b"), 120_000_000)
    assert len(sample.params) == 10 and sample.numel == 116_133_888


def test_headers_are_plain_c(tmp_path):
    """The boundary is a C ABI: both public headers compile as pedantic C11 and the struct sizes a
    foreign binding hard-codes are the ones the compiler sees."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi.c"
    src.write_text('#include "optengine.h"\n#include "gograd_host.h"\n'
                   "int main(void) { return sizeof(oe_tensor_desc) == 56 && sizeof(oe_adamw_hparams) == 48 &&\n"
                   "                        sizeof(oe_sgd_hparams) == 40 && sizeof(gg_sgd_options) == 24 &&\n"
                   "                        sizeof(oe_zero1_desc) == 320 && sizeof(gg_sgd_config) == 28 ? 0 : 1; }\n")
    exe = tmp_path / "abi"
    subprocess.run([cc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
