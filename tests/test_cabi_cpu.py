"""CPU: the shared library loads, exports every symbol the header declares, and the ctypes
table binds exactly those symbols.  No compute calls (there is no GPU here)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from cudnn_vsa_b200 import _cabi
from cudnn_vsa_b200.vsa import block_wo_padding_to_raster, raster_to_block_wo_padding, vsa_attention
from cudnn_vsa_b200.vsa_layout import Segment, build_vsa_layout

HEADER = Path(__file__).resolve().parent.parent / "include" / "vsa_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(vsa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 13
    lib = ctypes.CDLL(str(_cabi.LIB_PATH))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_cabi.SIGNATURES) == names
    assert _cabi.load().vsa_abi_version() >= 1
    assert _cabi.load().vsa_kv_mask_words(65) == 3


def test_header_argument_counts_match_the_binding():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    for name, (_, argtypes) in _cabi.SIGNATURES.items():
        args = re.search(rf"\b{name}\s*\((.*?)\)\s*;", text, flags=re.S).group(1).strip()
        count = 0 if args in ("", "void") else args.count(",") + 1
        assert count == len(argtypes), name


def test_public_entry_validation_happens_on_the_host():
    layout = build_vsa_layout([[Segment("video", (4, 4, 4), .5), Segment("text", 5)]], head_num=2)
    x = torch.zeros(layout.tokens, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="VSALayout"):
        vsa_attention(x, x, x, x, None)
    with pytest.raises(ValueError, match="VSA requires a gate tensor"):
        vsa_attention(x, x, x, None, layout)
    with pytest.raises(ValueError, match="identical shape"):
        vsa_attention(x, x, x[:-1], x, layout)
    with pytest.raises(ValueError, match="contiguous"):
        vsa_attention(x, x, x.transpose(0, 1).contiguous().transpose(0, 1), x, layout)
    with pytest.raises(ValueError, match="layout.tokens"):
        vsa_attention(x[:-1], x[:-1], x[:-1], x[:-1], layout)
    y = torch.zeros(layout.tokens, 3, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="VSALayout.head_num"):
        vsa_attention(y, y, y, y, layout)
    with pytest.raises(ValueError, match="CUDA BF16"):
        vsa_attention(x, x, x, x, layout)  # CPU tensors: no fallback
    with pytest.raises(ValueError, match="positive dimensions"):
        vsa_attention(x[:0], x[:0], x[:0], x[:0], layout)


def test_reorder_validation_order():
    raster = build_vsa_layout([[Segment("video", (4, 4, 4), .5)]], head_num=2)
    block = build_vsa_layout([[Segment("video", (4, 4, 4), .5)]], head_num=2, input_order="block")
    x = torch.zeros(block.tokens, 4)
    with pytest.raises(ValueError, match="input_order"):
        raster_to_block_wo_padding(x, vsa_layout=raster)
    with pytest.raises(ValueError, match="one tensor"):
        raster_to_block_wo_padding([x], vsa_layout=block)
    with pytest.raises(ValueError, match="shape"):
        raster_to_block_wo_padding(x[:-1], vsa_layout=block)
    with pytest.raises(ValueError, match="nonempty"):
        raster_to_block_wo_padding(x[:, :0], vsa_layout=block)
    with pytest.raises(ValueError, match="dtype"):
        raster_to_block_wo_padding(x.to(torch.complex64), vsa_layout=block)
    with pytest.raises(ValueError, match="CUDA"):
        block_wo_padding_to_raster(x, vsa_layout=block)


def test_selftest_entry_rejects_bad_arguments_on_the_host():
    lib = _cabi.load()
    # Null status, non-positive limit, limit beyond the library's own one-second bound: all refused
    # before anything is launched (no GPU is needed for this).
    assert lib.vsa_selftest_wait_timeout(None, 1000, None) == 1
    dummy = ctypes.c_int32(0)
    pointer = ctypes.cast(ctypes.pointer(dummy), ctypes.c_void_p)
    assert lib.vsa_selftest_wait_timeout(pointer, 0, None) == 1
    assert lib.vsa_selftest_wait_timeout(pointer, 1 << 40, None) == 1
