"""Run the reference's own CUDA library (oracle/_ref/libcudaBERT_ref.so, built by
oracle/build_ref.py) on one batch and save its pooler output.  TEST INFRASTRUCTURE.

    python oracle/run_ref_cuda.py <weight_dir> <large 0|1> <inputs.npz> <out.npy>

Runs in a process of its own: the reference exits the process on any error
(cuda_bert/utils/common.h:58-65) and exports the same symbol names as the product library.
`inputs.npz` holds int32 ids, seg and (optionally) mask of shape [B, S].  Calls, unmodified, the
reference's init_model / Cuda_Bert / release_model (cuda_bert/cuda_bert.cu:26-70)."""
import ctypes
import os
import sys

import numpy as np
from numpy.ctypeslib import ndpointer


def main():
    wdir, large, inp, out = sys.argv[1], bool(int(sys.argv[2])), sys.argv[3], sys.argv[4]
    here = os.path.dirname(os.path.abspath(__file__))
    lib = ctypes.CDLL(os.path.join(here, "_ref", "libcudaBERT_ref.so"))
    lib.init_model.argtypes = [ctypes.c_bool, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_char_p]
    lib.init_model.restype = ctypes.c_void_p
    lib.release_model.argtypes = [ctypes.c_void_p]
    i32 = ndpointer(np.int32, flags="C_CONTIGUOUS")
    lib.Cuda_Bert.argtypes = [ctypes.c_void_p, ndpointer(np.float32, flags="C_CONTIGUOUS"), i32, i32, ctypes.c_int,
                              ctypes.c_int, ctypes.c_void_p]
    data = np.load(inp)
    ids = np.ascontiguousarray(data["ids"], np.int32)
    seg = np.ascontiguousarray(data["seg"], np.int32)
    mask = np.ascontiguousarray(data["mask"], np.int32) if "mask" in data.files else None
    B, S = ids.shape
    model = lib.init_model(large, 0, B, S, wdir.encode())
    H = 1024 if large else 768
    res = np.zeros((B, H), np.float32)
    lib.Cuda_Bert(model, res, ids, seg, B, S, None if mask is None else mask.ctypes.data_as(ctypes.c_void_p))
    np.save(out, res)
    lib.release_model(model)


if __name__ == "__main__":
    main()
