"""Forward pass of the reference's small classification network
(modelnet40_small.py:121-261, MCConv variant) on the library's ops: point
hierarchy by Poisson disk sampling, one Monte-Carlo convolution per level,
inference batch normalisation + leaky ReLU + Conv1x1 between the levels, a
two-layer head.  Weights come from the caller (synthetic.small_classifier_weights
in the tests and the benchmark); dropout is the identity at inference."""
import math

import torch

from . import mcconv, pc

KERAS_BN_EPS = 1e-3        # tf.keras.layers.BatchNormalization default epsilon
KERAS_LEAKY_ALPHA = 0.3    # tf.keras.layers.LeakyReLU default slope


# Level layouts: (sampling radii, feature sizes input -> per level -> head).
# 'script': modelnet40_small.py:121-261, 331 (four levels, the last radius
# 2 sqrt(3) leaves one point per cloud, two dense layers).  'three_level': three
# levels with radii 0.1 / 0.2 / sqrt(3), widths 128 / 256 / 1024 and a single
# 1024 -> 40 layer as head; sqrt(3) can leave several points per cloud, which are
# averaged before the head.
PRESETS = {
    'script': dict(radii=(0.1, 0.2, 0.4, 2 * math.sqrt(3)),
                   feature_sizes=(1, 128, 256, 512, 1024, 1024, 40), head_layers=2,
                   pool_before_head=False),
    'three_level': dict(radii=(0.1, 0.2, math.sqrt(3)), feature_sizes=(1, 128, 256, 1024, 40),
                        head_layers=1, pool_before_head=True),
}


class SmallClassifier:
  def __init__(self, weights, sample_radii, device, pool_before_head=False):
    self.pool_before_head = bool(pool_before_head)
    to = lambda a: torch.from_numpy(a).to(device)
    self.radii = [float(r) for r in sample_radii]
    self.convs = []
    for w1, b1, wf in weights["conv"]:
      cin = wf.shape[1] // w1.shape[2]
      self.convs.append(mcconv.MCConv(to(w1), to(b1), to(wf), cin))
    self.conv1x1 = [(to(w), to(b)) for w, b in weights["conv1x1"]]
    self.dense = [(to(w), to(b)) for w, b in weights["dense"]]
    # a freshly initialised batch normalisation in inference mode: mean 0,
    # variance 1, gamma 1, beta 0
    self.bn_scale = 1.0 / math.sqrt(1.0 + KERAS_BN_EPS)

  def _bn_act(self, x):
    return mcconv.scale_bias_activation_(x.contiguous(), self.bn_scale, None, KERAS_LEAKY_ALPHA)

  def forward(self, points, batch_ids, batch_size, features):
    cloud = pc.PointCloud(points, batch_ids, batch_size)
    hier = pc.PointHierarchy(cloud, self.radii, 'poisson')
    clouds = hier._point_clouds
    x = features
    last = len(self.convs) - 1
    for i, conv in enumerate(self.convs):
      x = conv.forward(x, clouds[i], clouds[i + 1], self.radii[i], keep_for_backward=False)
      if i < last:
        x = self._bn_act(x)
        x = mcconv.conv1x1(x, *self.conv1x1[i])
        x = self._bn_act(x)
    # return_sorted=True of the last convolution (modelnet40_small.py:249-254):
    # rows in ascending batch id; the last radius leaves one point per cloud
    if self.pool_before_head:
      x = mcconv.global_pool(x, clouds[-1], 'avg')
    else:
      order = torch.argsort(clouds[-1]._batch_ids.long(), stable=True)
      x = x[order].contiguous()
    x = self._bn_act(x)
    for w, b in self.dense[:-1]:
      x = self._bn_act(mcconv.conv1x1(x, w, b))
    return mcconv.conv1x1(x, *self.dense[-1])
