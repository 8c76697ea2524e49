"""ResNet-50 v1 in fp32 NCHW with random weights, as an operator graph that both the CPU
oracle and the device engine can run.

Architecture (the published one, batch norm folded into the convolutions' bias): 7x7 stride-2
stem to 64 channels + ReLU, 3x3 stride-2 max pool, then 3 + 4 + 6 + 3 bottleneck blocks
(1x1 -> 3x3 -> 1x1 with 4x expansion; the first block of a stage has a 1x1 projection
shortcut).  The stride of a stage sits in the block's FIRST 1x1 convolution and in the
projection (the original v1 placement), so every 3x3 convolution has stride 1 and takes the
Winograd path, every 1x1 the GEMM path.  Residual sum and its ReLU are separate Eltwise and
Activation operators, the way MACE's converter emits them.  Global average pool, 1000-way
FullyConnected.

Weights: He-normal (std sqrt(2 / fan_in)); bias N(0, 0.01); input uniform in [0, 1).
"""
import numpy as np

NUM_CLASSES = 1000
STAGES = ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2))  # bottleneck width, blocks, stride
RELU, NOOP = 1, 0


def _same(h, k, s):
    out = -(-h // s)
    return out, max((out - 1) * s + k - h, 0)


def build(seed=0, image=224, width_div=1):
    """Returns (nodes, weights).  nodes: dicts with op / name / inputs and the op's attributes;
    weights: name -> array.  width_div shrinks every channel count (tests use it to keep the
    CPU oracle fast); 1 is the real network."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nodes, weights = [], {}

    def conv(name, src, cin, cout, k, stride, act):
        fan_in = cin * k * k
        weights[name + "_w"] = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        weights[name + "_b"] = (rng.standard_normal(cout) * 0.01).astype(np.float32)
        nodes.append({"op": "conv", "name": name, "inputs": [src], "cin": cin, "cout": cout, "k": k,
                      "stride": stride, "act": act})
        return name

    c0 = 64 // width_div
    x = conv("conv1", "input", 3, c0, 7, 2, RELU)
    nodes.append({"op": "maxpool", "name": "pool1", "inputs": [x], "k": 3, "stride": 2})
    x, cin = "pool1", c0
    for si, (width, blocks, stride) in enumerate(STAGES):
        w = width // width_div
        for b in range(blocks):
            p = "res%d%c" % (si + 2, ord("a") + b)
            s = stride if b == 0 else 1
            if b == 0:
                short = conv(p + "_branch1", x, cin, 4 * w, 1, s, NOOP)
            else:
                short = x
            y = conv(p + "_branch2a", x, cin, w, 1, s, RELU)
            y = conv(p + "_branch2b", y, w, w, 3, 1, RELU)
            y = conv(p + "_branch2c", y, w, 4 * w, 1, 1, NOOP)
            nodes.append({"op": "add", "name": p + "_sum", "inputs": [short, y]})
            nodes.append({"op": "relu", "name": p, "inputs": [p + "_sum"]})
            x, cin = p, 4 * w
    nodes.append({"op": "avgpool", "name": "pool5", "inputs": [x]})
    weights["fc_w"] = (rng.standard_normal((NUM_CLASSES, cin, 1, 1)) * np.sqrt(2.0 / cin)).astype(np.float32)
    weights["fc_b"] = (rng.standard_normal(NUM_CLASSES) * 0.01).astype(np.float32)
    nodes.append({"op": "fc", "name": "fc", "inputs": ["pool5"], "cin": cin})
    return nodes, weights


def random_images(batch, seed, image=224):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.random((batch, 3, image, image), dtype=np.float32)


def shapes(nodes, batch, image):
    """name -> (N, C, H, W) of every activation."""
    out = {"input": (batch, 3, image, image)}
    for n in nodes:
        _, c, h, w = out[n["inputs"][0]]
        if n["op"] == "conv":
            ho, _ = _same(h, n["k"], n["stride"])
            wo, _ = _same(w, n["k"], n["stride"])
            out[n["name"]] = (batch, n["cout"], ho, wo)
        elif n["op"] == "maxpool":
            ho, _ = _same(h, n["k"], n["stride"])
            wo, _ = _same(w, n["k"], n["stride"])
            out[n["name"]] = (batch, c, ho, wo)
        elif n["op"] in ("add", "relu"):
            out[n["name"]] = (batch, c, h, w)
        elif n["op"] == "avgpool":
            out[n["name"]] = (batch, c, 1, 1)
        else:
            out[n["name"]] = (batch, NUM_CLASSES, 1, 1)
    return out


def macs_per_image(nodes, image=224):
    sh = shapes(nodes, 1, image)
    total = 0
    for n in nodes:
        if n["op"] == "conv":
            _, co, ho, wo = sh[n["name"]]
            total += co * ho * wo * n["cin"] * n["k"] * n["k"]
        elif n["op"] == "fc":
            total += n["cin"] * NUM_CLASSES
    return total


def activation_bytes(nodes, batch, image=224):
    """Compulsory traffic of one forward pass: every operator reads its inputs and writes its
    output once (fp32), plus the weights once."""
    sh = shapes(nodes, batch, image)
    total = 0
    for n in nodes:
        for i in n["inputs"]:
            total += 4 * int(np.prod(sh[i]))
        total += 4 * int(np.prod(sh[n["name"]]))
        if n["op"] == "conv":
            total += 4 * (n["cout"] * n["cin"] * n["k"] * n["k"] + n["cout"])
        elif n["op"] == "fc":
            total += 4 * (n["cin"] * NUM_CLASSES + NUM_CLASSES)
    return total


def oracle_forward(orc, nodes, weights, x, keep=False):
    """The CPU oracle through the whole graph (direct fp32 convolutions); returns the logits
    [N, 1000, 1, 1] (and every activation by name when keep is set)."""
    acts = {"input": x}
    for n in nodes:
        a = acts[n["inputs"][0]]
        if n["op"] == "conv":
            _, _, h, w = a.shape
            ho, wo, ph, pw = orc.calc_padding_and_output_size(h, w, n["k"], n["k"], (1, 1),
                                                              (n["stride"],) * 2, 1)
            y = orc.conv2d_f32(a, weights[n["name"] + "_w"], weights[n["name"] + "_b"], (n["stride"],) * 2,
                               (1, 1), (ph >> 1, pw >> 1), (ho, wo), n["act"])
        elif n["op"] == "maxpool":
            _, _, h, w = a.shape
            ho, wo, ph, pw = orc.calc_padding_and_output_size(h, w, n["k"], n["k"], (1, 1),
                                                              (n["stride"],) * 2, 1)
            y = orc.pooling_f32(a, (n["k"],) * 2, (n["stride"],) * 2, (1, 1), (ph >> 1, pw >> 1), (ho, wo), 2)
        elif n["op"] == "add":
            y = orc.eltwise_f32(a, acts[n["inputs"][1]], 0)
        elif n["op"] == "relu":
            y = orc.activation_f32(a, RELU)
        elif n["op"] == "avgpool":
            _, _, h, w = a.shape
            y = orc.pooling_f32(a, (h, w), (1, 1), (1, 1), (0, 0), (1, 1), 1)
        else:
            nb = a.shape[0]
            y = orc.gemv_f32(weights["fc_w"].reshape(NUM_CLASSES, -1), a.reshape(nb, -1), weights["fc_b"],
                             nb, NUM_CLASSES, n["cin"], False, True).reshape(nb, NUM_CLASSES, 1, 1)
        acts[n["name"]] = y
    return (acts["fc"], acts) if keep else acts["fc"]


def build_engine(hostapi, nodes, weights, batch, device=0, image=224):
    """Registers weights and operators with a HostEngine; the input tensor is "input", the
    logits "fc"."""
    eng = hostapi.HostEngine(device)
    eng.add_tensor("input", shape=(batch, 3, image, image), dtype=hostapi.DT_FLOAT)
    F = hostapi.DT_FLOAT
    for n in nodes:
        name, ins = n["name"], n["inputs"]
        if n["op"] == "conv":
            eng.add_tensor(name + "_w", weights[name + "_w"], is_weight=True)
            eng.add_tensor(name + "_b", weights[name + "_b"], is_weight=True)
            eng.op("Conv2D", name, [ins[0], name + "_w", name + "_b"], [name], T=F,
                   ints={"strides": [n["stride"]] * 2, "dilations": [1, 1]}, i={"padding": hostapi.SAME},
                   s={"activation": "RELU" if n["act"] == RELU else "NOOP"})
        elif n["op"] == "maxpool":
            eng.op("Pooling", name, ins, [name], T=F,
                   ints={"kernels": [n["k"]] * 2, "strides": [n["stride"]] * 2, "dilations": [1, 1]},
                   i={"padding": hostapi.SAME, "pooling_type": hostapi.MAX})
        elif n["op"] == "add":
            eng.op("Eltwise", name, ins, [name], T=F, i={"type": 0})
        elif n["op"] == "relu":
            eng.op("Activation", name, ins, [name], T=F, s={"activation": "RELU"})
        elif n["op"] == "avgpool":
            sh = shapes(nodes, batch, image)[ins[0]]
            eng.op("Pooling", name, ins, [name], T=F,
                   ints={"kernels": [sh[2], sh[3]], "strides": [1, 1], "dilations": [1, 1]},
                   i={"padding": hostapi.VALID, "pooling_type": hostapi.AVG})
        else:
            eng.add_tensor("fc_w", weights["fc_w"], is_weight=True)
            eng.add_tensor("fc_b", weights["fc_b"], is_weight=True)
            eng.op("FullyConnected", name, [ins[0], "fc_w", "fc_b"], [name], T=F)
    return eng
