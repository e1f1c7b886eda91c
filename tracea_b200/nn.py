"""torch.nn front end of the conv path: the reference's `TraceaConv2d` / `patch_conv2d`
(tracea-python/python/tracea/__init__.py:19-56), forward only.

Differences from the reference's module, all deliberate:
  * dilation > 1 is computed here (the reference falls back to PyTorch for it);
  * configurations the library does not compute (groups != 1, a padding_mode other than "zeros", string paddings)
    raise NotImplementedError instead of silently running PyTorch's own convolution: this package has no fallback
    path, and a caller should know which backend produced its numbers;
  * OIHW-contiguous weights are packed into the kernel's [K][R][S][C] layout once per weight version
    (`ops.prepack_conv2d_weight`) and then read in place on every call.
"""
import torch

from . import ops


class TraceaConv2d(torch.nn.Conv2d):
    """Drop-in for torch.nn.Conv2d on CUDA tensors (fp32 as TF32, fp16, bf16). The output takes the memory format of
    the input; channels-last inputs are consumed in place."""

    def _check(self):
        if self.groups != 1:
            raise NotImplementedError("TraceaConv2d: groups=%d is not supported (groups must be 1)" % self.groups)
        if self.padding_mode != "zeros":
            raise NotImplementedError("TraceaConv2d: padding_mode=%r is not supported" % self.padding_mode)
        if isinstance(self.padding, str):
            raise NotImplementedError("TraceaConv2d: padding=%r is not supported, pass integers" % (self.padding,))

    def _kernel_weight(self):
        w = self.weight.detach()
        vec = 16 // w.element_size()
        if w.stride(1) == 1 or w.shape[1] % vec != 0:
            return w            # already channels-last, or channel-padded per call inside the library
        key = (w._version, w.data_ptr(), w.dtype, w.device)
        cached = getattr(self, "_tracea_packed", None)
        if cached is None or cached[0] != key:
            cached = (key, ops.prepack_conv2d_weight(w))
            self._tracea_packed = cached
        return cached[1]

    def forward(self, x):
        self._check()
        bias = self.bias.detach() if self.bias is not None else None
        return ops.conv2d_nchw(x, self._kernel_weight(), bias, None, self.stride, self.padding, self.dilation, 1,
                               "bias" if bias is not None else None)


def patch_conv2d():
    """Replace torch.nn.Conv2d with TraceaConv2d for modules constructed afterwards
    (tracea-python/python/tracea/__init__.py:19-26)."""
    torch.nn.Conv2d = TraceaConv2d
