"""Drop-in for the reference's pybind module ``cpu_adam_op``.

Same three functions with the same positional signatures
(patrickstar/ops/csrc/adam/cpu_adam.cpp:751-756), but the tensors are CUDA
tensors and the update runs in the sm_100a kernel.  ``adam_update`` keeps the
reference's conventions: tensors are flat (``.view(-1)``), params / exp_avg /
exp_avg_sq are fp32 and updated in place, grads are fp16 or fp32 and read-only,
``loss_scale`` <= 0 means no unscale, the return value is 0.  Unlike the
reference, a failing call raises instead of being ignored.
"""
import ctypes as C

import torch

from ._lib import check, lib


def create_adam(optimizer_id, alpha=1e-3, betta1=0.9, betta2=0.999, eps=1e-8, weight_decay=0.0,
                adamw_mode=True, should_log=False):
    check(lib.ps_adam_create(optimizer_id, alpha, betta1, betta2, eps, weight_decay, int(adamw_mode),
                             int(should_log)), "create_adam")
    return 0


def destroy_adam(optimizer_id):
    check(lib.ps_adam_destroy(optimizer_id), "destroy_adam")
    return 0


def adam_update(optimizer_id, step, lr, beta1, beta2, epsilon, weight_decay, bias_correction, params,
                grads, exp_avg, exp_avg_sq, loss_scale, fp16_params_out=None):
    """``fp16_params_out`` (optional, not in the reference): fp16 tensor that
    receives half(params); may be ``grads`` itself, which is the chunk layout's
    convention (the gradient lives in the fp16 param's storage)."""
    for name, t in (("params", params), ("grads", grads), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
        if not t.is_cuda:
            raise TypeError("adam_update: %s must be a CUDA tensor (there is no CPU path)" % name)
        if not t.is_contiguous():
            # the reference silently updates a temporary copy here (cpu_adam.cpp:714-717)
            raise ValueError("adam_update: %s must be contiguous" % name)
    if params.dtype != torch.float32 or exp_avg.dtype != torch.float32 or exp_avg_sq.dtype != torch.float32:
        raise TypeError("adam_update: params, exp_avg and exp_avg_sq must be fp32")
    if grads.dtype not in (torch.float16, torch.float32):
        raise TypeError("adam_update: grads must be fp16 or fp32")
    n = params.size(0) if params.dim() else 1  # the reference passes params_c.size(0)
    out_ptr = None
    if fp16_params_out is not None:
        if fp16_params_out.dtype != torch.float16 or not fp16_params_out.is_cuda:
            raise TypeError("adam_update: fp16_params_out must be a CUDA fp16 tensor")
        out_ptr = fp16_params_out.data_ptr()
    with torch.cuda.device(params.device):
        stream = C.c_void_p(torch.cuda.current_stream(params.device).cuda_stream)
        check(lib.ps_adam_update(optimizer_id, step, lr, beta1, beta2, epsilon, weight_decay,
                                 int(bool(bias_correction)), params.data_ptr(), grads.data_ptr(),
                                 exp_avg.data_ptr(), exp_avg_sq.data_ptr(), n,
                                 int(grads.dtype == torch.float16), float(loss_scale), out_ptr, stream),
              "adam_update")
    return 0
