"""Synthetic quantized MobileNet-v1 1.0 (224x224, uint8 NHWC, random weights): the layer
list, seeded weights, per-tensor quantization, a CPU-oracle forward pass and a builder for
the C++ host engine.  No dataset or checkpoint is involved: weights are He-normal floats
quantized per tensor, activation ranges come from a small seeded calibration batch."""
import numpy as np

# (kind, out_channels, stride): stem conv, then 13 x (depthwise 3x3, pointwise 1x1)
PW_OUT = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
DW_STRIDE = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]
NUM_CLASSES = 1000


def macs_per_image():
    total, h, c = 112 * 112 * 27 * 32, 112, 32
    for o, s in zip(PW_OUT, DW_STRIDE):
        h = h // s
        total += h * h * c * 9 + h * h * c * o
        c = o
    return total + 1024 * NUM_CLASSES


def _quantize_weights(orc, w):
    scale, zp = orc.adjust_range(w.min(), w.max(), True)  # non_zero as the CPU converter does
    return orc.quantize(w, scale, zp), scale, zp


def _same_pad(h, k, s):
    out = (h - 1) // s + 1
    total = max(0, (out - 1) * s + k - h)
    return out, total


def _calib_conv(x, w_real, stride):
    """Float NHWC conv (OHWI weights) for calibration, SAME padding with MACE's split."""
    n, h, wd, c = x.shape
    o, kh, kw, _ = w_real.shape
    ho, ph = _same_pad(h, kh, stride)
    wo, pw = _same_pad(wd, kw, stride)
    xp = np.zeros((n, h + ph, wd + pw, c), np.float32)
    xp[:, ph >> 1:(ph >> 1) + h, pw >> 1:(pw >> 1) + wd] = x
    cols = []
    for i in range(kh):
        for j in range(kw):
            cols.append(xp[:, i:i + (ho - 1) * stride + 1:stride, j:j + (wo - 1) * stride + 1:stride])
    col = np.concatenate(cols, axis=-1).reshape(-1, kh * kw * c)
    return (col @ w_real.reshape(o, -1).T).reshape(n, ho, wo, o)


def _calib_dw(x, w_real, stride):
    """Float NHWC depthwise 3x3 (HWIM weights, multiplier 1)."""
    n, h, wd, c = x.shape
    ho, ph = _same_pad(h, 3, stride)
    wo, pw = _same_pad(wd, 3, stride)
    xp = np.zeros((n, h + ph, wd + pw, c), np.float32)
    xp[:, ph >> 1:(ph >> 1) + h, pw >> 1:(pw >> 1) + wd] = x
    y = np.zeros((n, ho, wo, c), np.float32)
    for i in range(3):
        for j in range(3):
            y += xp[:, i:i + (ho - 1) * stride + 1:stride, j:j + (wo - 1) * stride + 1:stride] * \
                w_real[i, j, :, 0]
    return y


def build(orc, seed=0, calib_images=2, image=224):
    """Returns the list of layer dicts with quantized weights, int32 biases and activation
    quantization.  Activations: zero point 0, scale = min(6, observed max) / 255."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x_q = rng.integers(0, 256, size=(calib_images, image, image, 3), dtype=np.uint8)
    s_in, zp_in = np.float32(1.0 / 255.0), 0
    x_real = x_q.astype(np.float32) * s_in
    layers = []

    def finish(kind, name, w, y_fn, stride, fan_in, **extra):
        nonlocal x_real, s_in
        w_f = rng.normal(0.0, np.sqrt(2.0 / fan_in), size=w).astype(np.float32)
        w_q, s_f, zp_f = _quantize_weights(orc, w_f)
        w_real = (w_q.astype(np.float32) - zp_f) * s_f
        nbias = extra["channels"]
        bias_scale = np.float32(s_in * s_f)
        bias = np.rint(rng.normal(0.0, 0.01, size=nbias) / bias_scale).astype(np.int32)
        y = y_fn(x_real, w_real, stride) + bias.astype(np.float32) * bias_scale
        top = float(min(6.0, y.max()))
        if top <= 0:
            top = 6.0
        s_out = np.float32(top / 255.0)
        layers.append(dict(kind=kind, name=name, w=w_q, s_f=s_f, zp_f=zp_f, bias=bias,
                           bias_scale=bias_scale, stride=stride, s_in=s_in, zp_in=0,
                           s_out=s_out, zp_out=0))
        x_real = np.clip(np.rint(y / s_out), 0, 255).astype(np.float32) * s_out
        s_in = s_out

    finish("conv", "stem", (32, 3, 3, 3), _calib_conv, 2, 27, channels=32)
    c = 32
    for k, (o, s) in enumerate(zip(PW_OUT, DW_STRIDE)):
        finish("dw", "dw%d" % (k + 1), (3, 3, c, 1), _calib_dw, s, 9, channels=c)
        finish("conv", "pw%d" % (k + 1), (o, 1, 1, c), _calib_conv, 1, c, channels=o)
        c = o
    # global average pool keeps scale / zero point
    layers.append(dict(kind="pool", name="pool", kernel=x_real.shape[1], s_in=s_in, zp_in=0))
    pooled = x_real.mean(axis=(1, 2), keepdims=True)
    w_f = rng.normal(0.0, np.sqrt(2.0 / 1024), size=(NUM_CLASSES, 1, 1, 1024)).astype(np.float32)
    w_q, s_f, zp_f = _quantize_weights(orc, w_f)
    bias_scale = np.float32(s_in * s_f)
    bias = np.rint(rng.normal(0.0, 0.01, size=NUM_CLASSES) / bias_scale).astype(np.int32)
    logits = pooled.reshape(-1, 1024) @ ((w_q.astype(np.float32) - zp_f) * s_f).reshape(NUM_CLASSES, 1024).T
    logits = logits + bias.astype(np.float32) * bias_scale
    s_out, zp_out = orc.adjust_range(logits.min(), logits.max(), False)
    layers.append(dict(kind="fc", name="fc", w=w_q, s_f=s_f, zp_f=zp_f, bias=bias,
                       bias_scale=bias_scale, s_in=s_in, zp_in=0, s_out=s_out, zp_out=zp_out))
    return layers


def random_images(batch, seed, image=224):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, 256, size=(batch, image, image, 3), dtype=np.uint8)


def oracle_forward(orc, layers, x, keep=False):
    """The CPU oracle through the whole chain; returns uint8 logits [N, 1000] (and every
    intermediate activation when keep is set)."""
    acts = []
    for L in layers:
        n, h, w, c = x.shape
        if L["kind"] == "conv":
            o, kh, kw, _ = L["w"].shape
            ho, wo, ph, pw = orc.calc_padding_and_output_size(h, w, kh, kw, (1, 1),
                                                              (L["stride"],) * 2, 1)
            m, sh = orc.output_multiplier_and_shift(L["s_f"], L["s_in"], L["s_out"])
            x = orc.conv2d_u8(x, L["w"], L["bias"], (L["stride"],) * 2, (ph, pw), (ho, wo),
                              L["zp_in"], L["zp_f"], m, sh, L["zp_out"])
        elif L["kind"] == "dw":
            ho, wo, ph, pw = orc.calc_padding_and_output_size(h, w, 3, 3, (1, 1),
                                                              (L["stride"],) * 2, 1)
            m, sh = orc.output_multiplier_and_shift(L["s_in"], L["s_f"], L["s_out"])
            x = orc.dwconv_u8(x, L["w"], L["bias"], (L["stride"],) * 2, (1, 1), (ph >> 1, pw >> 1),
                              (ho, wo), L["zp_in"], L["zp_f"], m, sh, L["zp_out"])
        elif L["kind"] == "pool":
            x = orc.avgpool_u8(x, (h, w), (1, 1), (0, 0), (1, 1))
        else:  # fc: the Gemv delegator's float-multiplier rule
            mult = np.float32(L["s_f"]) * np.float32(L["s_in"]) / np.float32(L["s_out"])
            x = orc.gemv_u8(L["w"].reshape(1, NUM_CLASSES, -1), x.reshape(n, -1), L["bias"], n,
                            NUM_CLASSES, 1024, L["zp_f"], L["zp_in"], mult, L["zp_out"], True)
            x = x.reshape(n, NUM_CLASSES)
        if keep:
            acts.append(x)
    return (x, acts) if keep else x


def build_engine(hostapi, layers, batch, device=0, image=224):
    """Registers the weights and the operator chain with a HostEngine (tensors named like
    the layers; the input tensor is "input", the logits "fc")."""
    eng = hostapi.HostEngine(device)
    eng.add_tensor("input", shape=(batch, image, image, 3), dtype=hostapi.DT_UINT8,
                   scale=1.0 / 255.0, zero_point=0)
    prev = "input"
    for L in layers:
        name = L["name"]
        if L["kind"] in ("conv", "dw", "fc"):
            eng.add_tensor(name + "_w", L["w"], scale=L["s_f"], zero_point=L["zp_f"], is_weight=True)
            eng.add_tensor(name + "_b", L["bias"], scale=L["bias_scale"], zero_point=0, is_weight=True)
        if L["kind"] == "conv":
            eng.op("Conv2D", name, [prev, name + "_w", name + "_b"], [name],
                   out_quant=[(L["s_out"], L["zp_out"])],
                   ints={"strides": [L["stride"]] * 2, "dilations": [1, 1]},
                   i={"padding": hostapi.SAME})
        elif L["kind"] == "dw":
            eng.op("DepthwiseConv2d", name, [prev, name + "_w", name + "_b"], [name],
                   out_quant=[(L["s_out"], L["zp_out"])],
                   ints={"strides": [L["stride"]] * 2, "dilations": [1, 1]},
                   i={"padding": hostapi.SAME})
        elif L["kind"] == "pool":
            eng.op("Pooling", name, [prev], [name],
                   ints={"kernels": [L["kernel"]] * 2, "strides": [1, 1], "dilations": [1, 1]},
                   i={"padding": hostapi.VALID, "pooling_type": hostapi.AVG})
        else:
            eng.op("FullyConnected", name, [prev, name + "_w", name + "_b"], [name],
                   out_quant=[(L["s_out"], L["zp_out"])])
        prev = name
    return eng
