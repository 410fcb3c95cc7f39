"""Offline weight preparation: bf16 ``[n, k]`` weights -> the byte layouts the matmul plans read,
stored in one tagged container file.

    python -m mircuda_b200.weight_prep --format nvfp4 --input weights.pt --output weights.mirw

``weights.pt`` is a ``torch.save``d mapping of names to 2-D tensors; every tensor is converted
on ``cuda:0`` with the library's own kernels (the same entry points the plans' callers use, so
a prepared file and an on-the-fly conversion are the same bytes). Formats:

``mxfp8``         E4M3 codes ``[n, k]`` + E8M0 scales per 32 in 128 x 4 atoms (mircuda_mxfp8_tc_*)
``nvfp4``         E2M1 codes ``[n, k/2]`` + UE4M3 scales per 16 in 128 x 4 atoms + fp32 global
                  (mircuda_fp4_*, mircuda_b200_nvfp4_vector_*, the grouped NVFP4 plans)
``marlin_nvfp4``  the same quantisation, codes in Marlin tiles, scales re-encoded and the global
                  compensated (sys/native/marlin/repack.cu:105-140) (mircuda_marlin_nvfp4_*)
``int4_g128``     symmetric int4 codes ``[n, k/2]`` + f16 scales per 128 (mircuda_b200_w4a16_*)

Container: ``b"MIRB200W"``, u32 layout version, u32 header bytes, a JSON header (format, layout
version, per-tensor name / dtype / shape / offset / bytes), then the blobs, each 256-byte
aligned. A reader refuses a layout version it does not know.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import struct
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib, dense, plans

MAGIC = b"MIRB200W"
LAYOUT_VERSION = 1
FORMATS = ("mxfp8", "nvfp4", "marlin_nvfp4", "int4_g128")
_ALIGN = 256
_DTYPES = {"uint8": torch.uint8, "float16": torch.float16, "float32": torch.float32}


class UnknownLayout(ValueError):
    """The file is not a prepared-weight container of a layout version this reader knows."""


@dataclass
class PreparedWeight:
    """One weight in one format: named byte tensors plus the logical shape."""
    format: str
    n: int
    k: int
    tensors: dict = field(default_factory=dict)


def _pointer(tensor: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(tensor.data_ptr())


def _nvfp4_row_major(stream, weight: torch.Tensor):
    """NVFP4 codes, row-major UE4M3 scales [n, k/16] and the device global scale."""
    n, k = weight.shape
    library = _lib.load()
    handle = plans._stream_handle(stream)
    with torch.cuda.stream(stream):
        codes = torch.empty(n * k // 2, dtype=torch.uint8, device=weight.device)
        scales = torch.empty(n * k // 16, dtype=torch.uint8, device=weight.device)
        global_scale = torch.zeros(1, dtype=torch.float32, device=weight.device)
    plans._check(library.mircuda_b200_nvfp4_global_scale(_pointer(weight), n * k,
                                                         _pointer(global_scale), handle))
    plans._check(library.mircuda_b200_nvfp4_quantize_rows_bf16(
        _pointer(weight), _pointer(global_scale), _pointer(codes), _pointer(scales), n, k, handle))
    return codes, scales, global_scale


def prepare(stream, weight: torch.Tensor, format: str) -> PreparedWeight:
    """Converts one bf16 ``[n, k]`` CUDA tensor. Shapes a format cannot take raise
    ``InvalidMatmulShape``."""
    if format not in FORMATS:
        raise ValueError(f"unknown format {format!r}; one of {FORMATS}")
    if weight.dim() != 2 or not weight.is_cuda:
        raise plans.InvalidMatmulShape("weights are 2-D CUDA tensors")
    weight = weight.to(torch.bfloat16).contiguous()
    n, k = weight.shape
    library = _lib.load()
    handle = plans._stream_handle(stream)
    result = PreparedWeight(format, n, k)
    if format == "mxfp8":
        if k % 32 != 0:
            raise plans.InvalidMatmulShape("k must be a multiple of 32")
        with torch.cuda.stream(stream):
            codes = torch.empty(n * k, dtype=torch.uint8, device=weight.device)
            scales = torch.zeros(plans.scale_bytes(n, k // 32), dtype=torch.uint8, device=weight.device)
        plans.mxfp8_quantize_bf16(stream, weight, codes, scales)
        result.tensors = {"codes": codes.view(n, k), "scales": scales}
    elif format == "nvfp4":
        codes, scales, global_scale = plans.nvfp4_quantize_bf16(stream, weight)
        result.tensors = {"codes": codes, "scales": scales, "global_scale": global_scale}
    elif format == "marlin_nvfp4":
        if n % 64 != 0 or k % 64 != 0:
            raise plans.InvalidMatmulShape("n and k must be multiples of 64")
        codes, scales, global_scale = _nvfp4_row_major(stream, weight)
        with torch.cuda.stream(stream):
            tiles = torch.empty_like(codes)
            prepared = torch.empty_like(scales)
            prepared_global = torch.zeros(1, dtype=torch.float32, device=weight.device)
            maximum = torch.zeros(1, dtype=torch.int32, device=weight.device)
        plans._check(library.mircuda_marlin_nvfp4_repack(handle, _pointer(codes), _pointer(tiles), 1, n, k))
        plans._check(library.mircuda_marlin_nvfp4_prepare_scales(
            handle, _pointer(scales), None, _pointer(global_scale), _pointer(prepared),
            _pointer(prepared_global), _pointer(maximum), 1, n, k))
        result.tensors = {"tiles": tiles, "scales": prepared, "global_scale": prepared_global}
    else:
        with torch.cuda.stream(stream):
            packed, scales = dense.quantize_int4(weight)
        result.tensors = {"codes": packed, "scales": scales}
    stream.synchronize()
    return result


def save(path, weights: dict) -> None:
    """Writes ``{name: PreparedWeight}`` (all of one format) as one container file."""
    formats = {prepared.format for prepared in weights.values()}
    if len(formats) != 1:
        raise ValueError("one container holds one format")
    entries, blobs, offset = [], [], 0
    for name, prepared in weights.items():
        for part, tensor in prepared.tensors.items():
            host = tensor.detach().cpu().contiguous()
            data = host.numpy().tobytes()
            offset = (offset + _ALIGN - 1) // _ALIGN * _ALIGN
            entries.append({"weight": name, "part": part, "dtype": str(host.dtype).split(".")[1],
                            "shape": list(host.shape), "offset": offset, "bytes": len(data)})
            blobs.append((offset, data))
            offset += len(data)
    header = json.dumps({
        "layout_version": LAYOUT_VERSION, "format": formats.pop(),
        "weights": {name: {"n": p.n, "k": p.k} for name, p in weights.items()},
        "tensors": entries}).encode()
    preamble = len(MAGIC) + 8 + len(header)
    base = (preamble + _ALIGN - 1) // _ALIGN * _ALIGN
    with open(path, "wb") as file:
        file.write(MAGIC + struct.pack("<II", LAYOUT_VERSION, len(header)) + header)
        for start, data in blobs:
            file.seek(base + start)
            file.write(data)


def load(path, device="cpu") -> dict:
    """Reads a container back into ``{name: PreparedWeight}`` with tensors on ``device``."""
    with open(path, "rb") as file:
        raw = file.read()
    if raw[:len(MAGIC)] != MAGIC:
        raise UnknownLayout("not a prepared-weight container")
    version, header_bytes = struct.unpack_from("<II", raw, len(MAGIC))
    if version != LAYOUT_VERSION:
        raise UnknownLayout(f"layout version {version}; this reader knows {LAYOUT_VERSION}")
    start = len(MAGIC) + 8
    header = json.loads(raw[start:start + header_bytes])
    if header.get("layout_version") != LAYOUT_VERSION or header.get("format") not in FORMATS:
        raise UnknownLayout("header does not match the preamble")
    base = (start + header_bytes + _ALIGN - 1) // _ALIGN * _ALIGN
    weights = {name: PreparedWeight(header["format"], shape["n"], shape["k"])
               for name, shape in header["weights"].items()}
    for entry in header["tensors"]:
        begin = base + entry["offset"]
        if begin + entry["bytes"] > len(raw):
            raise UnknownLayout("truncated container")
        dtype = _DTYPES[entry["dtype"]]
        array = np.frombuffer(raw, dtype=np.uint8, count=entry["bytes"], offset=begin).copy()
        tensor = torch.from_numpy(array).view(dtype).view(entry["shape"]).to(device)
        weights[entry["weight"]].tensors[entry["part"]] = tensor
    return weights


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--format", required=True, choices=FORMATS)
    parser.add_argument("--input", required=True, help="torch.save'd mapping of names to 2-D tensors")
    parser.add_argument("--output", required=True)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("weight preparation runs the library's CUDA kernels: no GPU is visible")
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    source = torch.load(args.input, map_location="cpu", weights_only=True)
    prepared = {name: prepare(stream, tensor.cuda(), args.format)
                for name, tensor in source.items() if tensor.dim() == 2}
    save(args.output, prepared)
    print(json.dumps({"format": args.format, "layout_version": LAYOUT_VERSION,
                      "weights": len(prepared), "output": args.output}))


if __name__ == "__main__":
    main()
