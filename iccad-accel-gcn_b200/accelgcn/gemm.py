"""Dense feature transform Z = H @ W of a GCN layer (agcn_gemm_tf32): fp32 in and out, TF32
multiply on the sm_100a tensor cores.  Only 128 x 128 weights are built."""
from __future__ import annotations

from . import _lib


def gemm_tf32(h, w, out=None, stream=None):
    """h [m, 128] fp32 CUDA (row stride may exceed 128), w [128, 128] fp32 contiguous -> z [m, 128]."""
    import torch
    lib = _lib.load()
    if not (h.is_cuda and w.is_cuda and h.dtype == torch.float32 and w.dtype == torch.float32):
        raise TypeError("gemm_tf32 needs float32 CUDA tensors")
    if h.dim() != 2 or w.dim() != 2 or h.shape[1] != w.shape[0] or h.stride(1) != 1 or not w.is_contiguous():
        raise ValueError("gemm_tf32: h must be [m, k] with unit column stride, w contiguous [k, n]")
    z = out if out is not None else torch.empty((h.shape[0], w.shape[1]), dtype=torch.float32, device=h.device)
    s = stream if stream is not None else torch.cuda.current_stream(h.device)
    with torch.cuda.device(h.device):
        _lib.check(lib.agcn_gemm_tf32(h.data_ptr(), h.stride(0) if h.shape[0] > 1 else h.shape[1], w.data_ptr(),
                                      z.data_ptr(), z.stride(0) if z.shape[0] > 1 else z.shape[1],
                                      h.shape[0], w.shape[0], w.shape[1], s.cuda_stream))
    return z


def gemm_tf32_async(h, w, out, status, stream=None):
    """The same product enqueued without waiting or allocating (agcn_gemm_tf32_async).  `status` is an
    int32 CUDA tensor of one element the caller owns: 0 after the stream has been synchronised unless
    a bounded wait inside the kernel ran out (1 producer, 2 MMA issuer, 3 epilogue)."""
    import torch
    lib = _lib.load()
    s = stream if stream is not None else torch.cuda.current_stream(h.device)
    with torch.cuda.device(h.device):
        _lib.check(lib.agcn_gemm_tf32_async(h.data_ptr(), h.stride(0) if h.shape[0] > 1 else h.shape[1], w.data_ptr(),
                                            out.data_ptr(), out.stride(0) if out.shape[0] > 1 else out.shape[1],
                                            h.shape[0], w.shape[0], w.shape[1], status.data_ptr(), s.cuda_stream))
    return out


def selftest_timeout(h, w, out, stream=None) -> int:
    """Runs the kernel's failure path on purpose (agcn_gemm_tf32_selftest_timeout) and returns the
    status code of the call: ERR_CUDA when the starved wait ran out and the kernel left cleanly."""
    import torch
    lib = _lib.load()
    s = stream if stream is not None else torch.cuda.current_stream(h.device)
    with torch.cuda.device(h.device):
        return lib.agcn_gemm_tf32_selftest_timeout(h.data_ptr(), h.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0),
                                                   h.shape[0], s.cuda_stream)


def gcn_fused_layer(indptr, indices, vals, z_in, w, m_rows, out=None, status=None, stream=None):
    """Z2[r] = relu(A[r, :] @ Z1) @ W for the first m_rows rows of a CSR matrix, all of at most 32
    nonzeros (agcn_gcn_fused_layer): the activations stay in shared memory between the gather and the
    tensor-core product.  z_in [n_cols, 128], w [128, 128] contiguous fp32 CUDA tensors."""
    import torch
    lib = _lib.load()
    if not (z_in.is_contiguous() and w.is_contiguous() and z_in.shape[1] == 128 and tuple(w.shape) == (128, 128)):
        raise ValueError("gcn_fused_layer: z_in must be contiguous [n_cols, 128] and w contiguous [128, 128]")
    dev = z_in.device
    z = out if out is not None else torch.empty((m_rows, 128), dtype=torch.float32, device=dev)
    st = status if status is not None else torch.zeros(1, dtype=torch.int32, device=dev)
    s = stream if stream is not None else torch.cuda.current_stream(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.agcn_gcn_fused_layer(indptr.data_ptr(), indices.data_ptr(), vals.data_ptr(), z_in.data_ptr(),
                                            w.data_ptr(), z.data_ptr(), int(m_rows), int(z_in.shape[0]), st.data_ptr(), s.cuda_stream))
    if status is None:
        s.synchronize()
        if int(st.item()) != 0:
            raise _lib.AccelGcnError(_lib.ERR_CUDA, f"agcn_gcn_fused_layer: status {int(st.item())} (1-3: a pipeline wait ran out; 4: column id out of range)")
    return z
