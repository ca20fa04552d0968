"""Build and load ``libmegacute_b200.so`` (the CUDA kernel + C ABI of include/megacute_b200.h).

The library is compiled in-tree with nvcc for sm_100a only.  There is no fallback: if the library
is missing or does not load, every entry point of the runtime raises.
"""

from __future__ import annotations

import ctypes
import os
import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
# MEGACUTE_B200_CHECK=1 selects the self-checking build (-DMK_CHECK: the kernel verifies the state of its shared-memory
# barriers before it arms or releases them and reports instead of going on; csrc/mk_device.cuh check_phase), a library
# file of its own beside the normal one.
CHECK_BUILD = os.environ.get("MEGACUTE_B200_CHECK") == "1"
LIB_PATH = pathlib.Path(os.environ.get("MEGACUTE_B200_LIB", PKG / ("libmegacute_b200_check.so" if CHECK_BUILD else "libmegacute_b200.so")))
# Relocatable device code: each op body is its own translation unit so that ptxas allocates its
# registers independently (csrc/ops.cuh says why).  -maxrregcount is the cap of an 11-warp CTA
# (three warps share one SM sub-partition's 16 K registers); callees in other translation units do
# not see the kernel's __launch_bounds__.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-rdc=true",
              "-maxrregcount=168", "-shared", "-Xcompiler", "-fPIC"]

ST_WORDS = 16
MAX_PTRS = 12


class OpDesc(ctypes.Structure):
    """mk_op_desc (256 bytes)."""
    _fields_ = [("kind", ctypes.c_int32), ("flags", ctypes.c_int32), ("i", ctypes.c_int32 * 22),
                ("f", ctypes.c_float * 4), ("ptr", ctypes.c_uint64 * MAX_PTRS), ("ld", ctypes.c_int32 * MAX_PTRS)]


class Caps(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("sm_count", "cc_major", "cc_minor", "max_smem_optin", "kernel_smem",
                                              "kernel_threads", "kernel_regs", "reserved")]


assert ctypes.sizeof(OpDesc) == 256

# name -> (restype, argtypes); every symbol include/megacute_b200.h declares
_P = ctypes.c_void_p
_I32P = ctypes.POINTER(ctypes.c_int32)
SYMBOLS = {
    "mk_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "mk_last_cuda_error": (ctypes.c_char_p, []),
    "mk_query": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(Caps)]),
    "mk_program_create": (ctypes.c_int, [ctypes.c_int, _P, ctypes.c_int, _P, ctypes.c_int, _P, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_P)]),
    "mk_program_set_ops": (ctypes.c_int, [_P, _P, ctypes.c_int, _P]),
    "mk_launch": (ctypes.c_int, [_P, _P]),
    "mk_program_set_timeout": (ctypes.c_int, [_P, ctypes.c_uint64]),
    "mk_program_status": (ctypes.c_int, [_P, _P, _I32P]),
    "mk_program_reset": (ctypes.c_int, [_P, _P]),
    "mk_program_epoch": (ctypes.c_int, [_P]),
    "mk_program_tcgen05_ops": (ctypes.c_int, [_P]),
    "mk_program_tcgen05_attention_ops": (ctypes.c_int, [_P]),
    "mk_program_packed_bytes": (ctypes.c_longlong, [_P]),
    "mk_program_refresh_weights": (ctypes.c_int, [_P, ctypes.c_void_p]),
    "mk_program_read_counters": (ctypes.c_int, [_P, _I32P, ctypes.c_int]),
    "mk_program_read_trace": (ctypes.c_int, [_P, _P, ctypes.c_size_t]),
    "mk_program_clear_trace": (ctypes.c_int, [_P, _P]),
    "mk_program_poke_wait": (ctypes.c_int, [_P, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "mk_program_destroy": (None, [_P]),
    "mk_launch_noalloc": (ctypes.c_int, [ctypes.c_int, _P, ctypes.c_int, _P, ctypes.c_int, _P, ctypes.c_int, _P, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, _P, _I32P]),
    "mk_noalloc_status": (ctypes.c_int, [ctypes.c_int, _P, _I32P]),
    "mk_argmax": (ctypes.c_int, [_P, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, _P, _P]),
}


def sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "megacute_b200.h"]


def needs_build() -> bool:
    return needs_build_of(LIB_PATH)


def needs_build_of(path: pathlib.Path) -> bool:
    return not path.exists() or any(s.stat().st_mtime > path.stat().st_mtime for s in sources())


def build(force: bool = False, verbose: bool = False, check: bool | None = None) -> pathlib.Path:
    """Compile the library with nvcc (cross-compiles without a GPU).  `check`: the -DMK_CHECK build (default: the
    one this process loads)."""
    check = CHECK_BUILD if check is None else check
    out = LIB_PATH if check == CHECK_BUILD else PKG / ("libmegacute_b200_check.so" if check else "libmegacute_b200.so")
    if not force and not needs_build_of(out):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, *(["-DMK_CHECK"] if check else []), "-o", str(out), *[str(f) for f in sorted(CSRC.glob("*.cu"))]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return out


_lib = None


def load():
    """The loaded library.  Raises if it has not been built (no CPU fallback exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            if os.environ.get("MEGACUTE_B200_AUTOBUILD", "1") == "1" and (CSRC / "megakernel.cu").exists():
                build()
            else:
                raise RuntimeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as e; e.build()'`")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class MegakernelError(RuntimeError):
    pass


class MegakernelTimeout(MegakernelError):
    """A device-side wait exceeded its limit; the launch ended with an error status."""


def check(rc: int, what: str = ""):
    if rc == 0:
        return
    lib = load()
    msg = lib.mk_strerror(rc).decode()
    if rc in (-1, -2):                   # CUDA errors and argument errors carry a detail message
        detail = lib.mk_last_cuda_error().decode()
        if detail:
            msg += ": " + detail
    raise MegakernelError(f"{what}: {msg}" if what else msg)
