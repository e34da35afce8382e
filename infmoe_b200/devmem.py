"""Raw device-memory reads for callers that hold plain device pointers."""
import numpy as np


def read_device(ptr: int, n: int, dtype) -> np.ndarray:
    """Copies n elements of `dtype` from a raw device pointer into a new numpy array (blocking)."""
    from cuda.bindings import runtime as rt

    buf = np.empty(n, dtype)
    (err,) = rt.cudaDeviceSynchronize()
    assert int(err) == 0, err
    (err,) = rt.cudaMemcpy(buf.ctypes.data, ptr, buf.nbytes, rt.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(err) == 0, err
    return buf
