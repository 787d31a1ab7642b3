"""The C-ABI library without a GPU: it loads, exports every declared symbol, and its
host-side argument checks answer before anything would be launched."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "b200moe.h"


@pytest.fixture(scope="module")
def lib():
    from b200moe import _lib

    if not _lib.library_path().exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location(
            "b200moe_build", REPO / "b300-moe-decode-fastpath_b200" / "build.py"
        )
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        module.build_library()
    return _lib.load()


def declared_functions() -> list[str]:
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface() -> None:
    names = declared_functions()
    for required in ("b200moe_forward", "b200moe_routing", "b200moe_gather",
                     "b200moe_gate_up_swiglu", "b200moe_down", "b200moe_combine",
                     "b200moe_scratch_bytes", "b200moe_build_info", "b200moe_abi_version"):
        assert required in names


def test_library_exports_every_declared_symbol(lib) -> None:
    from b200moe import _lib

    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/b200moe.h but not exported"
        assert name in _lib.EXPORTS, name


def test_build_info_attests_sm100a_and_no_fallback(lib) -> None:
    from b200moe import _lib

    info = _lib.build_info()
    assert info["compiled_architecture"] == "sm_100a"
    assert info["uses_fallback"] is False
    assert info["nvfp4_compiled"] is True
    assert "tcgen05" in info["bf16_grouped_gemm_provider"]
    assert lib.b200moe_abi_version() == _lib.ABI_VERSION
    assert lib.b200moe_nvfp4_available() == 1


def test_args_struct_matches_the_header_field_order() -> None:
    from b200moe._lib import B200MoeArgs

    text = HEADER.read_text()
    opening = "typedef struct B200MoeArgs {"
    body = text[text.index(opening) + len(opening): text.index("} B200MoeArgs;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields: list[str] = []
    for statement in body.split(";"):
        statement = statement.strip()
        if not statement:
            continue
        names = statement.split(",")
        first = names[0].split()[-1].lstrip("*")
        fields.append(first)
        fields.extend(n.strip().lstrip("*") for n in names[1:])
    assert fields == [name for name, _ in B200MoeArgs._fields_]
    assert ctypes.sizeof(B200MoeArgs) % 8 == 0


def test_python_constants_match_the_header() -> None:
    """Flags, status bits, tuning knobs and limits of the bindings are the header's."""

    from b200moe import _lib

    text = HEADER.read_text()
    defines = {
        name: int(value.rstrip("uU"), 0)
        for name, value in re.findall(
            r"^#define\s+B200MOE_(\w+)\s+\(?(-?(?:0[xX][0-9a-fA-F]+|\d+)[uU]?)\)?", text, re.M)
    }
    checked = 0
    for name, value in vars(_lib).items():
        if name.startswith(("FLAG_", "STATUS_", "TUNE_")) and isinstance(value, int):
            assert defines.get(name) == value, (name, value, defines.get(name))
            checked += 1
    assert checked >= 20
    # every flag, status bit and knob of the header has its Python name, and no two flags
    # or two knobs share a value
    for prefix in ("FLAG_", "STATUS_", "TUNE_"):
        names = [n for n in defines if n.startswith(prefix)]
        assert all(hasattr(_lib, n) for n in names), [n for n in names if not hasattr(_lib, n)]
        values = [defines[n] for n in names]
        assert len(set(values)) == len(values), prefix
    assert _lib.EP_MAX_WORLD == defines["EP_MAX_WORLD"]
    assert _lib.STATIC_ROUTING_MAX_ASSIGNMENTS == defines["STATIC_ROUTING_MAX_ASSIGNMENTS"]


def test_scratch_bytes_and_host_side_errors(lib) -> None:
    from b200moe import _lib

    small = _lib.scratch_bytes(1, 2, 8, 4096, 14336)
    large = _lib.scratch_bytes(64, 2, 8, 4096, 14336)
    assert 0 < small < large
    # partial rows dominate: 8 slices x rows x H x 4 bytes
    assert large >= 8 * 128 * 4096 * 4
    size = ctypes.c_size_t()
    assert lib.b200moe_scratch_bytes(1, 3, 8, 64, 64, ctypes.byref(size)) == -2   # K=3
    assert lib.b200moe_scratch_bytes(1, 2, 300, 64, 64, ctypes.byref(size)) == -2  # E>256
    assert lib.b200moe_scratch_bytes(1, 2, 8, 60, 64, ctypes.byref(size)) == -3    # H%8
    assert lib.b200moe_scratch_bytes(1, 2, 8, 64, 64, None) == -1
    assert lib.b200moe_forward(None, None) == -1
    args = _lib.B200MoeArgs()
    args.num_tokens, args.top_k, args.num_experts = 4, 3, 8
    args.hidden_size = args.intermediate_size = 64
    assert lib.b200moe_forward(ctypes.byref(args), None) == -2
    assert "top" in _lib.error_string(-2).lower() or "shape" in _lib.error_string(-2).lower()
    with pytest.raises(ValueError):
        _lib.check(-3, "probe")


def test_header_is_plain_c_and_links_from_c(lib, tmp_path) -> None:
    """The boundary is a C ABI: the header must compile as C99 (and as C++), and a C
    program must link against the library and call it with nothing but the header."""

    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    from b200moe import _lib

    source = tmp_path / "abi_check.c"
    source.write_text(
        '#include <stddef.h>\n#include <string.h>\n#include "b200moe.h"\n'
        "int main(void) {\n"
        "  B200MoeArgs args; size_t bytes = 0; char info[1024];\n"
        "  memset(&args, 0, sizeof args);\n"
        "  if (b200moe_abi_version() != B200MOE_ABI_VERSION) return 1;\n"
        "  if (b200moe_scratch_bytes(64, 2, 8, 4096, 14336, &bytes) != 0 || bytes == 0) return 2;\n"
        "  if (b200moe_scratch_bytes(64, 3, 8, 4096, 14336, &bytes) != B200MOE_E_SHAPE) return 3;\n"
        "  if (b200moe_forward(NULL, NULL) != B200MOE_E_NULL) return 4;\n"
        "  if (b200moe_build_info(info, sizeof info) <= 0 || !strstr(info, \"sm_100a\")) return 5;\n"
        "  if (b200moe_nvfp4_available() != 1) return 6;\n"
        "  return 0;\n}\n"
    )
    include = str(HEADER.parent)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                    "-I", include, str(source)], check=True)
    if shutil.which("g++"):
        subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++",
                        "-I", include, str(source)], check=True)
    library = _lib.library_path()
    binary = tmp_path / "abi_check"
    subprocess.run(["gcc", "-std=c99", "-I", include, str(source), "-o", str(binary),
                    f"-L{library.parent}", "-l:" + library.name,
                    f"-Wl,-rpath,{library.parent}"], check=True)
    result = subprocess.run([str(binary)], capture_output=True, text=True)
    assert result.returncode == 0, (result.returncode, result.stderr)
