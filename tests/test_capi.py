"""The C-ABI library loads and exports every symbol include/mynah_b200.h
declares; no compute call is made (this runs without a GPU)."""
import os
import re
import subprocess

from mynah_tts_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mynah_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(mynah_(?:cuda|b200|backend)_\w+)\s*\(", text))
    names -= {n for n in names if n.endswith("_fn")}
    return names


def test_header_declares_the_seam_symbols():
    names = declared_functions()
    # the symbols src/backend.c:105-135 of the reference binds for its CUDA device
    for sym in ("mynah_backend_cuda_open mynah_cuda_upload mynah_cuda_download mynah_cuda_sync "
                "mynah_cuda_snake_dev mynah_cuda_gelu_dev mynah_cuda_layer_norm_dev "
                "mynah_cuda_residual_add_dev mynah_cuda_matmul_dev mynah_cuda_sgemm_dev "
                "mynah_cuda_dev_alloc mynah_cuda_dev_free mynah_cuda_h2d mynah_cuda_d2h "
                "mynah_cuda_matvec_dev mynah_cuda_gelu_inplace mynah_cuda_residual_inplace "
                "mynah_cuda_layer_norm_inplace mynah_cuda_matmul_to_dev mynah_cuda_matmul_d2d "
                "mynah_cuda_im2col mynah_cuda_conv1d mynah_cuda_gelu_host mynah_cuda_gelu_host_f64 "
                "mynah_cuda_matmul_graph").split():
        assert sym in names, sym
    # the resident-attention ops of src/backend.h:135-179
    for sym in ("mynah_cuda_self_attention_dev mynah_cuda_cross_attention_dev mynah_cuda_argmax_dev "
                "mynah_cuda_copy_dev mynah_cuda_batch_begin").split():
        assert sym in names, sym


def test_library_exports_every_declared_symbol():
    lib = capi.bind(capi.load_library())
    declared = declared_functions()
    assert declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None
    out = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], capture_output=True, text=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    assert declared <= exported
    # nothing but the declared ABI leaks out of the library
    assert {e for e in exported if not e.startswith("_")} == declared


def test_reference_seam_build_links_against_this_library():
    """oracle/_ref/libmynah_ref_b200.so -- the reference's graph.c and backend.c (CUDA branch)
    -- resolves every mynah_cuda_* symbol it binds from libmynah_b200.so (no compute here)."""
    import ctypes
    from oracle import oracle as O
    if not O.have_ref("b200"):
        import pytest
        pytest.skip("compiled reference absent")
    lib = ctypes.CDLL(O.REF_SO["b200"])          # RTLD_NOW: fails on any unresolved symbol
    assert hasattr(lib, "ref_backend_light_up") and hasattr(lib, "ref_decoder_run")
