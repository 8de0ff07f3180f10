"""CPU restatement of the reference's batch augmentation (src/augmentation.c).

TEST INFRASTRUCTURE ONLY: imported by tests/ and by bench.py's CPU-baseline
leg, never by the shipped package.

Pinned against the reference's compiled code: tests/test_augmentation_oracle.py
compares it with fixtures written by tests/golden/make_augmentation_golden.py
from oracle/_ref/libvithost.so (data_augmentation_apply itself).  Everything
is float32 arithmetic in the reference's order of operations; the only values
that can differ from the C code are those that pass through libm
(cosf / sinf / logf), by an ulp.

Random numbers: splitmix64 (augmentation.c:8-13).  Because the state advances
by a constant per draw, draw number k of a stream is a pure function of the
start state, which is what lets the device version compute any pixel's noise
independently; this restatement draws sequentially like the C code.
"""
import numpy as np

MASK = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
F = np.float32
PI_F = F(3.14159265358979323846)

FIELDS = ["max_shift_pixels", "max_rotation_degrees", "max_scale_delta",
          "max_brightness_delta", "max_contrast_delta",
          "noise_standard_deviation", "erasing_probability",
          "erasing_max_side_fraction", "erasing_value", "minimum_value",
          "maximum_value"]


def mix(state):
    """Output of splitmix64 for an already advanced state (augmentation.c:9-12)."""
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


class Stream:
    def __init__(self, state):
        self.state = state & MASK

    def bits(self):
        self.state = (self.state + GOLDEN) & MASK
        return mix(self.state)

    def unit(self):
        """augmentation.c:15-17."""
        return (F(self.bits() >> 40) + F(0.5)) / F(16777216.0)

    def symmetric(self, magnitude):
        """augmentation.c:19-21."""
        return F(magnitude) * (F(2.0) * self.unit() - F(1.0))

    def index_below(self, limit):
        """augmentation.c:28-30."""
        return self.bits() % limit


def geometric_enabled(a):
    return (a["max_shift_pixels"] > 0 or a["max_rotation_degrees"] > 0 or
            a["max_scale_delta"] > 0)


def enabled(a):
    """data_augmentation_enabled, augmentation.c:169-176."""
    return bool(geometric_enabled(a) or a["max_brightness_delta"] > 0 or
                a["max_contrast_delta"] > 0 or
                a["noise_standard_deviation"] > 0 or
                a["erasing_probability"] > 0)


def valid(a, same_buffer):
    """Argument checks of data_augmentation_apply, augmentation.c:182-198."""
    return not (a["max_shift_pixels"] < 0 or a["max_rotation_degrees"] < 0 or
                a["max_scale_delta"] < 0 or a["max_scale_delta"] >= 1 or
                a["max_brightness_delta"] < 0 or a["max_contrast_delta"] < 0 or
                a["max_contrast_delta"] >= 1 or
                a["noise_standard_deviation"] < 0 or
                a["erasing_probability"] < 0 or a["erasing_probability"] > 1 or
                a["erasing_max_side_fraction"] < 0 or
                a["erasing_max_side_fraction"] > 1 or
                (geometric_enabled(a) and same_buffer))


def affine(image, shift_y, shift_x, angle, scale):
    """apply_affine_transform + bilinear sampling with edge padding
    (augmentation.c:36-90).  image: [channels, height, width] float32."""
    channels, height, width = image.shape
    inverse_cosine = F(np.cos(F(angle))) / F(scale)
    inverse_sine = F(np.sin(F(angle))) / F(scale)
    center_y = F(0.5) * F(height - 1)
    center_x = F(0.5) * F(width - 1)
    ys = (np.arange(height, dtype=F) - center_y - F(shift_y))[:, None]
    xs = (np.arange(width, dtype=F) - center_x - F(shift_x))[None, :]
    source_x = (inverse_cosine * xs + inverse_sine * ys) + center_x
    source_y = (-inverse_sine * xs + inverse_cosine * ys) + center_y
    cy = np.clip(source_y, F(0), F(height - 1)).astype(F)
    cx = np.clip(source_x, F(0), F(width - 1)).astype(F)
    top = cy.astype(np.int64)
    left = cx.astype(np.int64)
    bottom = np.where(top + 1 < height, top + 1, top)
    right = np.where(left + 1 < width, left + 1, left)
    wy = cy - top.astype(F)
    wx = cx - left.astype(F)
    out = np.empty_like(image)
    one = F(1.0)
    for c in range(channels):
        plane = image[c]
        upper = plane[top, left] * (one - wx) + plane[top, right] * wx
        lower = plane[bottom, left] * (one - wx) + plane[bottom, right] * wx
        out[c] = upper * (one - wy) + lower * wy
    return out


def apply(a, state, source):
    """data_augmentation_apply (augmentation.c:178-229).  `a` maps FIELDS to
    numbers, source is [batch, channels, height, width] float32.  Returns
    (destination, new_state)."""
    a = {k: F(v) for k, v in a.items()}
    source = np.ascontiguousarray(source, dtype=F)
    batch, channels, height, width = source.shape
    stream = Stream(state)
    out = np.empty_like(source)
    clamps = a["minimum_value"] < a["maximum_value"]
    for s in range(batch):
        if geometric_enabled(a):
            shift_y = stream.symmetric(a["max_shift_pixels"])
            shift_x = stream.symmetric(a["max_shift_pixels"])
            angle = stream.symmetric(a["max_rotation_degrees"]) * PI_F / F(180.0)
            scale = F(1.0) + stream.symmetric(a["max_scale_delta"])
            image = affine(source[s], shift_y, shift_x, angle, scale)
        else:
            image = source[s].copy()
        if a["max_brightness_delta"] > 0 or a["max_contrast_delta"] > 0:
            contrast = F(1.0) + stream.symmetric(a["max_contrast_delta"])
            brightness = stream.symmetric(a["max_brightness_delta"])
            for c in range(channels):
                flat = image[c].reshape(-1)
                # Sequential float32 sum, as the C loop (augmentation.c:118-121).
                mean = np.cumsum(flat, dtype=F)[-1] / F(flat.size)
                image[c] = (mean + (image[c] - mean) * contrast) + brightness
        if a["noise_standard_deviation"] > 0:
            flat = image.reshape(-1)
            for i in range(flat.size):
                radius = np.sqrt(F(-2.0) * np.log(stream.unit()), dtype=F)
                normal = radius * F(np.cos(F(2.0) * PI_F * stream.unit()))
                flat[i] = flat[i] + a["noise_standard_deviation"] * normal
        if clamps:
            image = np.clip(image, a["minimum_value"], a["maximum_value"])
        if a["erasing_probability"] > 0:
            if not stream.unit() >= a["erasing_probability"]:
                max_h = int(max(F(1.0), a["erasing_max_side_fraction"] * F(height)))
                max_w = int(max(F(1.0), a["erasing_max_side_fraction"] * F(width)))
                erased_h = 1 + stream.index_below(max_h)
                erased_w = 1 + stream.index_below(max_w)
                top = stream.index_below(height - erased_h + 1)
                left = stream.index_below(width - erased_w + 1)
                image[:, top:top + erased_h, left:left + erased_w] = a["erasing_value"]
        out[s] = image
    return out, stream.state


def translate(source, shift_y, shift_x):
    """data_augmentation_translate (augmentation.c:231-245)."""
    source = np.ascontiguousarray(source, dtype=F)
    return np.stack([affine(image, F(shift_y), F(shift_x), F(0.0), F(1.0))
                     for image in source])
