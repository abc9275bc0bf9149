"""GGUF tensor-type and file-type tables.

Type ids, block sizes and bytes-per-block follow the GGUF specification; the
reference keeps the same tables in fs/ggml/type.go:250-295 (ids) and
fs/ggml/ggml.go:407-513 (block / type sizes).
"""
from __future__ import annotations

import enum


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ1_S = 19
    IQ4_NL = 20
    IQ3_S = 21
    IQ2_S = 22
    IQ4_XS = 23
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    IQ1_M = 29
    BF16 = 30
    TQ1_0 = 34
    TQ2_0 = 35
    MXFP4 = 39
    NVFP4 = 40
    Q1_0 = 41


# type -> (elements per block, bytes per block)
_LAYOUT: dict[GGMLType, tuple[int, int]] = {
    GGMLType.F32: (1, 4),
    GGMLType.F16: (1, 2),
    GGMLType.BF16: (1, 2),
    GGMLType.F64: (1, 8),
    GGMLType.I8: (1, 1),
    GGMLType.I16: (1, 2),
    GGMLType.I32: (1, 4),
    GGMLType.I64: (1, 8),
    GGMLType.Q4_0: (32, 18),
    GGMLType.Q4_1: (32, 20),
    GGMLType.Q5_0: (32, 22),
    GGMLType.Q5_1: (32, 24),
    GGMLType.Q8_0: (32, 34),
    GGMLType.Q8_1: (32, 36),
    GGMLType.Q2_K: (256, 84),
    GGMLType.Q3_K: (256, 110),
    GGMLType.Q4_K: (256, 144),
    GGMLType.Q5_K: (256, 176),
    GGMLType.Q6_K: (256, 210),
    GGMLType.Q8_K: (256, 292),
    GGMLType.IQ2_XXS: (256, 66),
    GGMLType.IQ2_XS: (256, 74),
    GGMLType.IQ3_XXS: (256, 98),
    GGMLType.IQ1_S: (256, 50),
    GGMLType.IQ4_NL: (32, 18),
    GGMLType.IQ3_S: (256, 110),
    GGMLType.IQ2_S: (256, 82),
    GGMLType.IQ4_XS: (256, 136),
    GGMLType.IQ1_M: (256, 56),
    GGMLType.TQ1_0: (256, 54),
    GGMLType.TQ2_0: (256, 66),
    GGMLType.MXFP4: (32, 17),
    GGMLType.NVFP4: (64, 36),
    GGMLType.Q1_0: (128, 18),
}


def block_size(t: int) -> int:
    return _LAYOUT[GGMLType(t)][0]


def type_size(t: int) -> int:
    return _LAYOUT[GGMLType(t)][1]


def row_bytes(t: int, n_elements: int) -> int:
    """Bytes needed for ``n_elements`` contiguous elements of type ``t``."""
    bs, ts = _LAYOUT[GGMLType(t)]
    if n_elements % bs:
        raise ValueError(f"{n_elements} elements is not a multiple of the {GGMLType(t).name} block ({bs})")
    return n_elements // bs * ts


def tensor_bytes(t: int, shape: tuple[int, ...]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return row_bytes(t, n)


class FileType(enum.IntEnum):
    """``general.file_type`` values (fs/ggml/type.go:12-56)."""

    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    MXFP4_MOE = 4  # value written by the gpt-oss converter (convert/convert_gptoss.go:47)
    Q8_0 = 7
    Q5_0 = 8
    Q5_1 = 9
    Q2_K = 10
    Q3_K_S = 11
    Q3_K_M = 12
    Q3_K_L = 13
    Q4_K_S = 14
    Q4_K_M = 15
    Q5_K_S = 16
    Q5_K_M = 17
    Q6_K = 18
    BF16 = 32


_FILE_TYPE_NAMES = {
    "F32": FileType.F32, "F16": FileType.F16, "BF16": FileType.BF16, "Q8_0": FileType.Q8_0,
    "Q4_0": FileType.Q4_0, "Q4_1": FileType.Q4_1, "Q5_0": FileType.Q5_0, "Q5_1": FileType.Q5_1,
    "Q2_K": FileType.Q2_K, "Q3_K_S": FileType.Q3_K_S, "Q3_K_M": FileType.Q3_K_M, "Q3_K_L": FileType.Q3_K_L,
    "Q4_K_S": FileType.Q4_K_S, "Q4_K_M": FileType.Q4_K_M, "Q5_K_S": FileType.Q5_K_S,
    "Q5_K_M": FileType.Q5_K_M, "Q6_K": FileType.Q6_K, "MXFP4": FileType.MXFP4_MOE,
}

# Targets accepted by `create --quantize` (fs/ggml/type.go:58-90).
QUANTIZE_TARGETS = ("F32", "F16", "BF16", "Q8_0", "Q4_K_S", "Q4_K_M")


def parse_file_type(name: str) -> FileType:
    try:
        return _FILE_TYPE_NAMES[name.upper()]
    except KeyError:
        raise ValueError(f"unsupported quantization type {name}") from None


def file_type_name(ft: int) -> str:
    for k, v in _FILE_TYPE_NAMES.items():
        if int(v) == int(ft):
            return k
    return "unknown"
