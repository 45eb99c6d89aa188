"""CPU-side checks of the drop-in boundary: the shared library loads without a GPU and exports
every function include/vearo_b200.h declares; device calls fail loudly (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "vearo_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|const char\*)\s+(vb_\w+)\s*\(", text)))


def test_header_declares_the_backend_ops_surface():
    names = declared_functions()
    # one entry point per BackendOps field (crates/vearo-core/src/tensor.rs:1111-1175) ...
    for op in ("add sub mul div matmul relu sum mean gelu softmax layernorm layernorm_backward embedding "
               "embedding_backward cross_entropy cross_entropy_backward conv2d conv2d_backward maxpool2d "
               "maxpool2d_backward avgpool2d avgpool2d_backward batchnorm batchnorm_backward fused_attention "
               "fused_attention_backward").split():
        assert "vb_" + op in names, op
    # ... the memory hooks, the host-side autograd helpers, the optimizer steps, data parallel
    for fn in ("alloc retain release write read relu_backward gelu_backward softmax_backward reduce_to accumulate "
               "adamw_step sgd_step clip_grad_norm opt_create opt_step dp_init dp_allreduce dp_finish").split():
        assert "vb_" + fn in names, fn


def test_library_loads_and_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    lib = C.CDLL(os.path.join(ROOT, "vearo_b200", "libvearo_b200.so"))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_no_silent_fallback_without_a_device():
    import vearo_b200 as vb
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(vb.VearoError):
        vb.init(0)
    lib = vb.lib()
    slot = C.c_uint32(0)
    assert lib.vb_alloc(16, 1, C.byref(slot)) != 0        # VB_ERR_NOT_INIT, not a host allocation
    assert b"vb_init" in lib.vb_last_error()


def test_product_never_imports_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "vearo_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("no CPU fallback", ""), os.path.join(dirpath, f)


def _split_args(arglist):
    """Top-level comma split of a C or Rust parameter list (no nested parentheses occur in either file)."""
    arglist = arglist.strip()
    if arglist in ("", "void"):
        return []
    return [a for a in (x.strip() for x in arglist.split(",")) if a]


def test_rust_binding_text_declares_exactly_the_header():
    """rust_shim/src/ffi.rs cannot be compiled where there is no rustc, so it is held to the header as text: the same set of
    functions, each with the same number of parameters."""
    header = open(os.path.join(ROOT, "include", "vearo_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    c_decl = {m.group(1): len(_split_args(m.group(2)))
              for m in re.finditer(r"\b(?:int|const char\*)\s+(vb_\w+)\s*\(([^)]*)\)\s*;", header)}
    rust = open(os.path.join(ROOT, "rust_shim", "src", "ffi.rs")).read()
    rust = re.sub(r"//[^\n]*", "", rust)
    r_decl = {m.group(1): len(_split_args(m.group(2)))
              for m in re.finditer(r"pub fn (vb_\w+)\s*\(([^)]*)\)", rust, flags=re.S)}
    assert sorted(c_decl) == sorted(r_decl), (sorted(set(c_decl) - set(r_decl)), sorted(set(r_decl) - set(c_decl)))
    wrong = {n: (c_decl[n], r_decl[n]) for n in c_decl if c_decl[n] != r_decl[n]}
    assert not wrong, wrong


def test_rust_shim_fills_every_backend_ops_field():
    """The shim's wrappers carry the names of the BackendOps fields (crates/vearo-core/src/tensor.rs:1111-1175) and of the hooks."""
    text = open(os.path.join(ROOT, "rust_shim", "src", "lib.rs")).read()
    for op in ("add sub mul div matmul relu sum mean gelu softmax layernorm layernorm_backward embedding embedding_backward "
               "cross_entropy cross_entropy_backward conv2d conv2d_backward maxpool2d maxpool2d_backward avgpool2d "
               "avgpool2d_backward batchnorm batchnorm_backward fused_attention fused_attention_backward").split():
        assert re.search(r"\b%s\b" % op, text), op
    for hook in ("b200_alloc", "b200_write", "b200_read", "b200_refcount_inc", "b200_refcount_dec", "register_backend_ops", "register_cuda_hooks"):
        assert hook in text, hook
