"""Host-side mirror of managan/codegen_tensor_products.py:64-101: the autograd functions Bee, Cow0
and Cow1 (and Ant16, :19-61) with the reference's argument and output order."""
import torch

from . import ops, ant16


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


class Ant16(torch.autograd.Function):
    """Mirror of managan/codegen_tensor_products.py:19-61: inputs x_0, x_1, x_2 followed by (P, left) pairs in
    the order 000,110,220, 011,101,121,211,111, 022,202,112,222,212; outputs y_0, y_1, y_2."""

    @staticmethod
    def forward(ctx, x_0, x_1, x_2, *pl):
        if len(pl) != 26:
            raise RuntimeError("Ant16 takes x_0, x_1, x_2 and thirteen (P, left) pairs")
        args = [t.contiguous() for t in (x_0, x_1, x_2, *pl)]
        ctx.save_for_backward(*args)
        x_0, x_1, x_2 = args[:3]
        pl = args[3:]
        o0, o1, c1, o2, c2 = pl[0:6], pl[6:14], pl[14:16], pl[16:24], pl[24:26]
        y_0, = ant16.ant16_o0(x_0, x_1, x_2, *o0)
        y_1, = ant16.ant16_o1(x_0, x_1, x_2, *o1)
        y_2, = ant16.ant16_o2(x_0, x_1, x_2, *o2)
        y_1c, y_2c = ant16.ant16_oc(x_1, x_2, *c1, *c2)
        return y_0, y_1 + y_1c, y_2 + y_2c

    @staticmethod
    def backward(ctx, dy_0, dy_1, dy_2):
        args = ctx.saved_tensors
        x_0, x_1, x_2 = args[:3]
        pl = args[3:]
        dy_0, dy_1, dy_2 = dy_0.contiguous(), dy_1.contiguous(), dy_2.contiguous()
        o0, o1, c1, o2, c2 = pl[0:6], pl[6:14], pl[14:16], pl[16:24], pl[24:26]
        oc = (*c1, *c2)
        dx0 = ant16.ant16_o0_backward(dy_0, *o0)
        dx1 = ant16.ant16_o1_backward(dy_1, *o1)
        dx2 = ant16.ant16_o2_backward(dy_2, *o2)
        dxc = ant16.ant16_oc_backward(dy_1, dy_2, *oc)
        dl0 = ant16.ant16_o0_backleft(x_0, x_1, x_2, dy_0, *o0[0::2])
        dl1 = ant16.ant16_o1_backleft(x_0, x_1, x_2, dy_1, *o1[0::2])
        dl2 = ant16.ant16_o2_backleft(x_0, x_1, x_2, dy_2, *o2[0::2])
        dlc = ant16.ant16_oc_backleft(x_1, x_2, dy_1, dy_2, *oc[0::2])
        dP0 = ant16.ant16_o0_wtsback(x_0, x_1, x_2, dy_0, *o0[1::2])
        dP1 = ant16.ant16_o1_wtsback(x_0, x_1, x_2, dy_1, *o1[1::2])
        dP2 = ant16.ant16_o2_wtsback(x_0, x_1, x_2, dy_2, *o2[1::2])
        dPc = ant16.ant16_oc_wtsback(x_1, x_2, dy_1, dy_2, *oc[1::2])

        def interleave(dP, dl):
            out = []
            for a, b in zip(dP, dl):
                out += [a, b]
            return out

        return (dx0[0] + dx1[0] + dx2[0], dx0[1] + dx1[1] + dx2[1] + dxc[0], dx0[2] + dx1[2] + dx2[2] + dxc[1],
                *interleave(dP0, dl0), *interleave(dP1, dl1), dPc[0], dlc[0], *interleave(dP2, dl2), dPc[1], dlc[1])
