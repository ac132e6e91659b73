"""Seeded synthetic samples for the padded vision-LM batch tests, and a writer for the reference
loader's on-disk format (include/imagenet_vlm.h:28-47: shard header, sample records, split index),
used only by tests/golden/make_golden.py to let the unmodified reference build the batches."""
import os
import struct

import numpy as np

H, W, C = 16, 32, 3          # two 16x16 patches per image; not square on purpose
T_MAX = 12
MEAN = (0.485, 0.456, 0.406)   # include/imagenet_vlm.h:23-24
STD = (0.229, 0.224, 0.225)


def make_samples(seed, n, version):
    """[(label, text ids, payload)], payload = uint8 [H,W,C] pixels (versions 1, 2) or float32
    [patches, patch_dim] (version 3).  Text lengths run from 1 to T_MAX-1 (the longest that fits), ids cover the byte range."""
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        length = (T_MAX - 1, 1, 6, 3, 9)[i % 5]
        text = rng.integers(0, 257, size=length).astype(np.int32)
        label = int(rng.integers(0, 1000))
        if version >= 3:
            payload = rng.standard_normal(((H // 16) * (W // 16), C * 256)).astype(np.float32)
        else:
            payload = rng.integers(0, 256, size=(H, W, C)).astype(np.uint8)
        out.append((label, text, payload))
    return out


def write_dataset(root, split, samples, version):
    """One shard `<split>-00001-of-00001.bin` plus `<split>.idx`."""
    body, entries = b"", []
    for local, (label, text, payload) in enumerate(samples):
        rec = struct.pack("<ii", label, len(text)) + text.astype("<i4").tobytes()
        if version >= 2:
            cap = b"caption %d" % local
            rec += struct.pack("<i", len(cap)) + cap
        rec += payload.tobytes()
        entries.append(struct.pack("<IIQHH", 0, local, len(body), len(text), label))
        body += rec
    header = struct.pack("<8i", 0x494D474E, version, H, W, C, len(samples), 0, 1) + bytes(32)
    with open(os.path.join(root, "%s-00001-of-00001.bin" % split), "wb") as f:
        f.write(header + body)
    with open(os.path.join(root, split + ".idx"), "wb") as f:
        f.write(struct.pack("<IIQ", 0x58444E49, 1, len(samples)) + b"".join(entries))
