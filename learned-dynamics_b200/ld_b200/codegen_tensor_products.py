"""Host-side mirror of managan/codegen_tensor_products.py:64-101: the autograd functions Bee, Cow0
and Cow1 with the reference's argument and output order."""
import torch

from . import ops


class Bee(torch.autograd.Function):
    @staticmethod
    def forward(ctx, l_0, l_1, l_2, r_0, r_1, r_2):
        args = [t.contiguous() for t in (l_0, l_1, l_2, r_0, r_1, r_2)]
        ctx.save_for_backward(*args)
        return tuple(ops.bee_fwd(*args))

    @staticmethod
    def backward(ctx, *dy):
        l_0, l_1, l_2, r_0, r_1, r_2 = ctx.saved_tensors
        dl = ops.bee_bw(True, r_0, r_1, r_2, dy)
        dr = ops.bee_bw(False, l_0, l_1, l_2, dy)
        return (*dl, *dr)


class Cow0(torch.autograd.Function):
    @staticmethod
    def forward(ctx, l_0, l_1, r_0, r_1):
        args = [t.contiguous() for t in (l_0, l_1, r_0, r_1)]
        ctx.save_for_backward(*args)
        return tuple(ops.cow_o0_fwd(*args))

    @staticmethod
    def backward(ctx, dy_000, dy_110):
        l_0, l_1, r_0, r_1 = ctx.saved_tensors
        dl = ops.cow_o0_bw(r_0, r_1, dy_000, dy_110)
        dr = ops.cow_o0_bw(l_0, l_1, dy_000, dy_110)
        return (*dl, *dr)


class Cow1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, l_0, l_1, r_0, r_1):
        args = [t.contiguous() for t in (l_0, l_1, r_0, r_1)]
        ctx.save_for_backward(*args)
        return tuple(ops.cow_o1_fwd(*args))

    @staticmethod
    def backward(ctx, dy_011, dy_101, dy_111):
        l_0, l_1, r_0, r_1 = ctx.saved_tensors
        dl = ops.cow_o1_bw(True, r_0, r_1, dy_011, dy_101, dy_111)
        dr = ops.cow_o1_bw(False, l_0, l_1, dy_011, dy_101, dy_111)
        return (*dl, *dr)
