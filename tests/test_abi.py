"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares;
compute entry points fail loudly (no CPU fallback)."""
import ctypes as C
import pathlib
import re

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def built_lib():
    from pssa_b200 import build
    return build.build()


def header_symbols():
    text = (ROOT / "include" / "pssa_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pssa_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    L = C.CDLL(str(built_lib))
    names = header_symbols()
    assert len(names) >= 13
    for name in names:
        assert hasattr(L, name), f"{name} declared in include/pssa_b200.h but not exported"


def test_python_binding_covers_the_header(built_lib):
    from pssa_b200 import _native
    assert sorted(_native.SIGNATURES) == header_symbols()


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = (ROOT / "include" / "pssa_b200.h").read_text()
    assert "src/backend.rs" in text and "src/gpu_batch.rs" in text and "src/cuda/stage_bounds.rs" in text


def test_oracle_is_not_reachable_from_the_product():
    for path in list((ROOT / "pssa_b200").rglob("*.py")) + list((ROOT / "pssa_b200" / "csrc").glob("*")) + \
            list((ROOT / "include").glob("*")):
        if path.is_file() and path.suffix in {".py", ".cu", ".hpp", ".cuh", ".h", ".cpp"}:
            body = path.read_text()
            assert "oracle" not in body.replace("no CPU fallback", ""), f"{path} mentions the oracle"


def test_context_creation_without_a_gpu_fails_loudly(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import pssa_b200
    with pytest.raises(pssa_b200.B200Error) as err:
        pssa_b200.B200Dispatch(0)
    assert err.value.status == 3 and "no CPU fallback" in str(err.value)


def test_rust_binding_source_declares_every_symbol_of_the_header_with_matching_arity():
    """rust/pssa_b200_sys.rs is source only (no Rust toolchain in the build image): at least hold it to the header --
    every declared symbol present, and the same number of parameters as the ctypes signature table that the GPU tests run."""
    from pssa_b200 import _native
    text = (ROOT / "rust" / "pssa_b200_sys.rs").read_text()
    block = text[text.index('extern "C" {'):]
    found = {}
    for m in re.finditer(r"pub fn (pssa_b200_[a-z0-9_]+)\s*\(", block):
        depth, i, params, start = 1, m.end(), 0, m.end()
        while depth:  # walk to the matching parenthesis, counting the commas at depth one
            ch = block[i]
            depth += ch in "(<" and not block[i - 1:i + 1] == "->"
            depth -= ch in ")>" and not block[i - 1:i + 1] == "->"
            if ch == "," and depth == 1 and block[i + 1:].lstrip()[:1] != ")":
                params += 1
            i += 1
        body = block[start:i - 1].strip()
        found[m.group(1)] = 0 if not body else params + 1
    assert sorted(found) == header_symbols()
    for name, (_, args) in _native.SIGNATURES.items():
        assert found[name] == len(args), f"{name}: {found[name]} parameters in Rust, {len(args)} in the ctypes table"
    arm = (ROOT / "rust" / "backend_b200.rs").read_text()
    for method in ("dispatch_gemm_into", "try_dispatch_gemm_into", "ssm_forward_resident", "ssm_forward", "memory_forward_after_ssm",
                   "memory_forward", "softplus_in_place", "invalidate_weights", "backend_label", "forward_inference", "prefill_inference",
                   "reset_recurrent_state", "copy_recurrent_state_to", "copy_recurrent_state_from", "set_loops", "set_memory_top_k"):
        assert f"pub fn {method}" in arm, method
