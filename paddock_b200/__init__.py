"""paddock_b200 - B200 (sm_100a) kernel pack for Paddock's quantized linear layer.

The product is the shared library ``libpaddock_b200.so`` (CUDA, C ABI declared
in ``include/paddock_pack.h``).  This package is the thin Python binding the
tests and the benchmark drive it through: a loader that performs the same
checks as the reference's ``crates/paddock-kernels/src/loader.rs`` and a
call-by-slot helper.  There is no CPU fallback: without the library, or on a
machine without a CUDA device, every compute entry point raises.
"""
from .pack import (KernelPack, PackError, Open, NotAPack, BadDescriptor, BadMagic, AbiMismatch,
                   NoKernelTable, BadKernelTable, MissingOp, LaunchError, SLOTS, lib_path, header_path)

__all__ = ["KernelPack", "PackError", "Open", "NotAPack", "BadDescriptor", "BadMagic", "AbiMismatch",
           "NoKernelTable", "BadKernelTable", "MissingOp", "LaunchError", "SLOTS", "lib_path", "header_path"]
