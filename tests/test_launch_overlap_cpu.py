"""Source check for kernels launched with programmatic stream serialisation: such a kernel may be
scheduled while the kernel before it on the stream is still running, so it has to execute a
dependency wait before it touches global memory. A kernel without the wait reads its input while
the producer is still writing it, and breaks the ordering of everything launched after it."""
import pathlib
import re

CSRC = pathlib.Path(__file__).resolve().parent.parent / "mircuda_b200" / "csrc"

# Kernels of files with overlapped launches that are themselves launched with plain <<< >>>.
PLAIN_LAUNCHES = {
    "nvfp4_amax_kernel", "nvfp4_finish_global_scale_kernel", "mxfp8_swizzle_scales_kernel",
    "dense_gemm_plain_kernel", "dense_gemm_kernel", "scaled_fp8_rows_kernel", "scaled_fp8_kernel",
}


def kernels_of(text):
    """(name, body) of every __global__ function of a source text."""
    found = []
    for match in re.finditer(r"__global__", text):
        header_end = text.find("{", match.end())
        header = text[match.end():header_end]
        header = re.sub(r"__launch_bounds__\s*\([^)]*(\([^)]*\))?[^)]*\)", " ", header)
        header = re.sub(r"__cluster_dims__\s*\([^)]*\)", " ", header)
        name = re.search(r"(\w+)\s*\(", header)
        depth, cursor = 0, header_end
        while True:
            if text[cursor] == "{":
                depth += 1
            elif text[cursor] == "}":
                depth -= 1
                if depth == 0:
                    break
            cursor += 1
        found.append((name.group(1), text[header_end:cursor]))
    return found


def test_every_overlapped_kernel_waits_for_its_dependency():
    checked = 0
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))):
        text = path.read_text()
        if "launch_after_dependency(" not in text and "ProgrammaticStreamSerialization" not in text:
            continue
        for name, body in kernels_of(text):
            if name in PLAIN_LAUNCHES:
                # make sure the exemption is still true: the kernel is launched with <<< >>>
                assert re.search(name + r"(<[^<>]*>)?\s*<<<", text), f"{path.name}: {name} is exempted but not launched plainly"
                continue
            assert "dependency_wait()" in body or "griddepcontrol.wait" in body, \
                f"{path.name}: {name} is launched overlapped but never waits"
            checked += 1
    assert checked >= 20


def test_plain_kernels_are_not_launched_overlapped():
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))):
        text = path.read_text()
        for name in PLAIN_LAUNCHES:
            assert not re.search(r"launch_after_dependency\(\s*" + name + r"\b", text), f"{path.name}: {name}"
