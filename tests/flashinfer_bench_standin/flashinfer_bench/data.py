"""`SupportedBindings` of the stand-in (kbench asks for TVM_FFI only when language == "cuda")."""
import enum


class SupportedBindings(enum.Enum):
    TVM_FFI = "tvm_ffi"
    TORCH = "torch"
