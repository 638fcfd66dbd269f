"""ResNet family with torchvision's parameter names (so checkpoints interchange).

The reference ships no model code and benchmarks ``torchvision.models.resnet50``
(examples/pytorch_benchmark.py:100); this module states the same network (He et al.,
v1.5: stride on the 3x3 convolution of a bottleneck) in a form that suits a B200:
activations are NHWC (channels_last), parameters may be bf16 views of an fp32 master
bucket, BatchNorm statistics stay fp32, and the 1x1 convolutions and the classifier, which
are plain GEMMs in NHWC, can run on the hand-written tcgen05 GEMM
(``bluefog_b200.ops.gemm``) when ``use_b200_gemm`` is set; the stride-1 3x3 convolutions can run as
implicit GEMMs on the tcgen05 kernel of ``bluefog_b200.ops.conv`` when ``use_b200_conv`` is set.
"""
import os
from typing import List, Optional, Type

import torch
import torch.nn as nn
import torch.nn.functional as F

from bluefog_b200.ops import fused_bn
from bluefog_b200.ops.fused_bn import bn_act as _bn_act
from bluefog_b200.ops.fused_pool import global_avgpool, maxpool3x3s2


def bn_act(x, bn, relu=True, residual=None, stats=None):
    # the batch counters of all layers are advanced together in ResNet.forward
    return _bn_act(x, bn, relu=relu, residual=residual, count_batches=False, stats=stats)


class MixedBatchNorm2d(nn.BatchNorm2d):
    """BatchNorm whose affine parameters may be bf16 while the running statistics stay fp32."""

    def forward(self, x):
        w, b = self.weight, self.bias
        if w is not None and w.dtype != torch.float32 and x.dtype == w.dtype:
            # cuDNN's mixed mode wants fp32 scale/shift with 16-bit activations
            w, b = w.float(), b.float()
        if (self.training and self.track_running_stats and self.num_batches_tracked is not None
                and not getattr(self, "external_batch_count", False)):
            self.num_batches_tracked.add_(1)
        momentum = 0.0 if self.momentum is None else self.momentum
        return F.batch_norm(x, self.running_mean if (not self.training or self.track_running_stats) else None,
                            self.running_var if (not self.training or self.track_running_stats) else None,
                            w, b, self.training or not self.track_running_stats, momentum, self.eps)


# BLUEFOG_B200_FUSE_BN_STATS=0: the BatchNorm after a tcgen05 1x1 convolution takes its own statistics pass
FUSE_BN_STATS = os.environ.get("BLUEFOG_B200_FUSE_BN_STATS", "1") != "0"


class Conv1x1(nn.Conv2d):
    """1x1 convolution; in NHWC with stride 1 it is the GEMM [N*H*W, Cin] x [Cin, Cout]; the strided
    shortcut convolutions take the implicit-GEMM kernel, which reads every second pixel."""

    def __init__(self, cin, cout, stride=1, use_b200_gemm=False):
        super().__init__(cin, cout, kernel_size=1, stride=stride, bias=False)
        self.use_b200_gemm = use_b200_gemm

    # "auto": GEMMs with at most this many rows (pixels) take the tcgen05 kernel; on a B200 it beats the
    # library from there down (batch 64: the 14x14 and 7x7 layers), above it the library is on par or ahead
    AUTO_MAX_ROWS = 16384

    def takes_b200_gemm(self, x):
        use = self.use_b200_gemm
        if use == "auto":
            use = x.shape[0] * x.shape[2] * x.shape[3] <= self.AUTO_MAX_ROWS
        return bool(use) and self.stride[0] == 1 and x.is_cuda and x.dtype == torch.bfloat16

    def forward(self, x):
        if self.takes_b200_gemm(x):
            from bluefog_b200.ops import gemm
            return gemm.conv1x1(x, self.weight)
        if self.use_b200_gemm is True and self.stride[0] == 2 and x.is_cuda and x.dtype == torch.bfloat16:
            from bluefog_b200.ops import conv
            return conv.conv2d(x, self.weight, 2, 0)       # strided reads inside the implicit-GEMM kernel
        return super().forward(x)

    def forward_fork_bn_act(self, x, bn, relu):
        """``(bn_act(self(x), bn), shortcut)`` for the first convolution of a block whose shortcut is the identity:
        the shortcut's gradient is added inside the input-gradient GEMM (``ops.gemm.conv1x1_fork``)."""
        from bluefog_b200.ops import gemm
        if (self.takes_b200_gemm(x) and torch.is_grad_enabled() and x.requires_grad
                and gemm.conv1x1_fork_supported(x, self.weight)):
            sums = None
            if bn.training and FUSE_BN_STATS and self.weight.shape[0] <= self.weight.shape[1]:
                sums = fused_bn.take_sums(x.device, self.weight.shape[0])
            y, shortcut = gemm.conv1x1_fork(x, self.weight, sums)
            return bn_act(y, bn, relu=relu, stats=sums), shortcut
        return self.forward_bn_act(x, bn, relu), x

    def forward_bn_act(self, x, bn, relu, residual=None):
        """``bn_act(self(x), bn, ...)``; on the tcgen05 path the GEMM epilogue also takes the batch statistics of
        its output, so the BatchNorm kernels read the activation once instead of twice."""
        # Only the channel-reducing convolutions (Cout <= Cin, the first of every bottleneck): their GEMM waits on
        # its input, so the epilogue has time for the sums (200704 x 256 -> 64: +3 us against a 13 us statistics
        # pass).  A channel-expanding product is bound by its epilogue and loses what the skipped pass saves
        # (200704 x 64 -> 256: +33 us against 31 us).
        if (self.takes_b200_gemm(x) and bn.training and FUSE_BN_STATS
                and self.weight.shape[0] <= self.weight.shape[1]):
            from bluefog_b200.ops import gemm
            if gemm.conv1x1_supported(x, self.weight) and self.weight.shape[0] % 8 == 0:
                sums = fused_bn.take_sums(x.device, self.weight.shape[0])
                return bn_act(gemm.conv1x1(x, self.weight, col_stats=sums), bn, relu=relu, residual=residual, stats=sums)
        return bn_act(self(x), bn, relu=relu, residual=residual)


class StemConv(nn.Conv2d):
    """The 7x7 / stride 2 / 3-channel stem convolution.  With ``space_to_depth`` it is evaluated as
    the equivalent 4x4 / stride 1 convolution over 2x2 pixel blocks (12 channels, padded to 16):
    three input channels leave tensor-core tiles almost empty, sixteen do not.  The parameter
    keeps its [64, 3, 7, 7] shape; the rearrangement of the (tiny) weight is part of the graph."""

    def __init__(self, space_to_depth=False, use_b200_conv=True):
        super().__init__(3, 64, kernel_size=7, stride=2, padding=3, bias=False)
        self.space_to_depth = space_to_depth
        self.use_b200_conv = use_b200_conv

    def forward(self, x):
        h, w = x.shape[2:]
        if self.space_to_depth and x.is_cuda and h % 2 == 0 and w % 2 == 0:
            return self.forward_space_to_depth(x)
        return super().forward(x)

    def space_to_depth_weight(self):
        """[64, 3, 7, 7] -> [64, 16, 4, 4] channels_last (kernel padded to 8x8, 2x2 blocks folded into channels)."""
        w8 = F.pad(self.weight, (0, 1, 0, 1))
        w12 = w8.view(64, 3, 4, 2, 4, 2).permute(0, 1, 3, 5, 2, 4).reshape(64, 12, 4, 4)
        return F.pad(w12, (0, 0, 0, 0, 0, 4)).contiguous(memory_format=torch.channels_last)

    def forward_space_to_depth(self, x):
        n, c, h, w = x.shape
        w16 = self.space_to_depth_weight()
        hb, wb = (h + 6) // 2, (w + 6) // 2
        xp = F.pad(x, (3, 3, 3, 3))
        xs = xp.reshape(n, 3, hb, 2, wb, 2).permute(0, 1, 3, 5, 2, 4).reshape(n, 12, hb, wb)
        xs = F.pad(xs, (0, 0, 0, 0, 0, 4)).contiguous(memory_format=torch.channels_last)
        return F.conv2d(xs, w16)

    def forward_from_raw(self, x):
        """The same convolution for an input that still is what the data loader delivered (fp32 or bf16, NCHW
        or NHWC, no gradient): padding, space-to-depth, cast and layout change happen in one kernel."""
        from bluefog_b200.common.basics import get_basics
        from bluefog_b200.ops import conv
        xs = get_basics().native.s2d_stem_input(x)
        if not self.use_b200_conv:
            return F.conv2d(xs, self.space_to_depth_weight())
        # four taps (one per filter row) over 64-value slices of four neighbouring pixels on the tcgen05 kernel
        return conv.stem_conv(xs, self.space_to_depth_weight())


class Downsample(nn.Sequential):
    """1x1 convolution + BatchNorm on the shortcut (children named "0" and "1" as in torchvision)."""

    def __init__(self, cin, cout, stride, use_b200_gemm):
        super().__init__(Conv1x1(cin, cout, stride, use_b200_gemm=use_b200_gemm), MixedBatchNorm2d(cout))

    def forward(self, x):
        return self[0].forward_bn_act(x, self[1], relu=False)


class Conv3x3(nn.Conv2d):
    """3x3 convolution (stride 1 or 2); with ``use_b200_conv`` it runs as an implicit GEMM on the tcgen05
    kernels of ``bluefog_b200.ops.conv`` (forward, input gradient and filter gradient), otherwise on the library."""

    def __init__(self, cin, cout, stride=1, use_b200_conv=False):
        super().__init__(cin, cout, kernel_size=3, stride=stride, padding=1, bias=False)
        self.use_b200_conv = use_b200_conv

    def forward(self, x):
        if self.use_b200_conv and x.is_cuda and x.dtype == torch.bfloat16:
            from bluefog_b200.ops import conv
            return conv.conv3x3(x, self.weight, self.stride[0])
        return super().forward(x)


def conv3x3(cin, cout, stride=1, use_b200_conv=False):
    return Conv3x3(cin, cout, stride, use_b200_conv=use_b200_conv)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, use_b200_gemm=False, use_b200_conv=False):
        super().__init__()
        self.conv1 = conv3x3(inplanes, planes, stride, use_b200_conv)
        self.bn1 = MixedBatchNorm2d(planes)
        self.relu = nn.ReLU(inplace=True)
        self.conv2 = conv3x3(planes, planes, 1, use_b200_conv)
        self.bn2 = MixedBatchNorm2d(planes)
        self.downsample = downsample

    def forward(self, x):
        xa, xb = fused_bn.split_for_two_uses(x)      # see Bottleneck.forward
        identity = xb if self.downsample is None else self.downsample(xb)
        out = bn_act(self.conv1(xa), self.bn1, relu=True)
        return bn_act(self.conv2(out), self.bn2, relu=True, residual=identity)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, use_b200_gemm=False, use_b200_conv=False):
        super().__init__()
        self.conv1 = Conv1x1(inplanes, planes, use_b200_gemm=use_b200_gemm)
        self.bn1 = MixedBatchNorm2d(planes)
        self.conv2 = conv3x3(planes, planes, stride, use_b200_conv)
        self.bn2 = MixedBatchNorm2d(planes)
        self.conv3 = Conv1x1(planes, planes * 4, use_b200_gemm=use_b200_gemm)
        self.bn3 = MixedBatchNorm2d(planes * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        # the block reads x twice (first convolution, shortcut); where x comes from a fused BatchNorm the two
        # gradients go there as a pair instead of being added by autograd
        xa, xb = fused_bn.split_for_two_uses(x)
        if xa is not x:
            identity = xb if self.downsample is None else self.downsample(xb)
            out = self.conv1.forward_bn_act(xa, self.bn1, relu=True)
        elif self.downsample is None:
            out, identity = self.conv1.forward_fork_bn_act(x, self.bn1, relu=True)
        else:
            identity = self.downsample(x)
            out = self.conv1.forward_bn_act(x, self.bn1, relu=True)
        out = bn_act(self.conv2(out), self.bn2, relu=True)
        return self.conv3.forward_bn_act(out, self.bn3, relu=True, residual=identity)


class ResNet(nn.Module):
    def __init__(self, block: Type[nn.Module], layers: List[int], num_classes: int = 1000,
                 use_b200_gemm: bool = False, zero_init_residual: bool = False, stem_space_to_depth: bool = True,
                 use_b200_conv: bool = False):
        super().__init__()
        self.inplanes = 64
        self.use_b200_gemm = use_b200_gemm
        self.use_b200_conv = use_b200_conv
        self.conv1 = StemConv(space_to_depth=stem_space_to_depth, use_b200_conv=bool(use_b200_conv))
        self.bn1 = MixedBatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(kernel_size=3, stride=2, padding=1)
        self.layer1 = self._make_layer(block, 64, layers[0])
        self.layer2 = self._make_layer(block, 128, layers[1], stride=2)
        self.layer3 = self._make_layer(block, 256, layers[2], stride=2)
        self.layer4 = self._make_layer(block, 512, layers[3], stride=2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        self._bn_modules = [m for m in self.modules() if isinstance(m, MixedBatchNorm2d)]
        for m in self._bn_modules:
            m.external_batch_count = True        # advanced together in forward()
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
        if zero_init_residual:
            for m in self.modules():
                if isinstance(m, Bottleneck):
                    nn.init.constant_(m.bn3.weight, 0)
                elif isinstance(m, BasicBlock):
                    nn.init.constant_(m.bn2.weight, 0)

    def _make_layer(self, block, planes, blocks, stride=1):
        downsample = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            downsample = Downsample(self.inplanes, planes * block.expansion, stride, self.use_b200_gemm)
        kw = dict(use_b200_gemm=self.use_b200_gemm, use_b200_conv=self.use_b200_conv)
        layers = [block(self.inplanes, planes, stride, downsample, **kw)]
        self.inplanes = planes * block.expansion
        for _ in range(1, blocks):
            layers.append(block(self.inplanes, planes, **kw))
        return nn.Sequential(*layers)

    def forward(self, x):
        raw_stem = (self.conv1.space_to_depth and x.is_cuda and x.dim() == 4 and not x.requires_grad
                    and self.conv1.weight.dtype == torch.bfloat16 and x.dtype in (torch.float32, torch.bfloat16)
                    and x.shape[1] == 3 and x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0)
        if not raw_stem:
            if x.is_cuda and x.dim() == 4:
                x = x.contiguous(memory_format=torch.channels_last)
            if x.dtype != self.conv1.weight.dtype:
                x = x.to(self.conv1.weight.dtype)
        if self.training:
            fused_bn.begin_step(x.device)          # one memset for the statistics scratch of all layers
            counters = [m.num_batches_tracked for m in self._bn_modules if m.num_batches_tracked is not None]
            if counters:
                torch._foreach_add_(counters, 1)     # one launch for the batch counters of all layers
        stem = self.conv1.forward_from_raw(x) if raw_stem else self.conv1(x)
        x = maxpool3x3s2(bn_act(stem, self.bn1, relu=True))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = global_avgpool(x)
        if self.use_b200_gemm is True and x.is_cuda and x.dtype == torch.bfloat16:
            from bluefog_b200.ops import gemm
            if gemm.available():
                return gemm.linear(x, self.fc.weight, self.fc.bias)
        return self.fc(x)


def resnet18(num_classes=1000, **kw):
    return ResNet(BasicBlock, [2, 2, 2, 2], num_classes, **kw)


def resnet34(num_classes=1000, **kw):
    return ResNet(BasicBlock, [3, 4, 6, 3], num_classes, **kw)


def resnet50(num_classes=1000, **kw):
    return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, **kw)


def resnet101(num_classes=1000, **kw):
    return ResNet(Bottleneck, [3, 4, 23, 3], num_classes, **kw)
