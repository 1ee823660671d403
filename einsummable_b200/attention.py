"""attention_t: descriptor of the fused attention chain (es_attention_t of the C ABI).

The reference has no such node: it stands for the five apply nodes its graph writer emits for
softmax(Q K^T + mask) V (src/einsummable/gwriter.cc:830-855, llama/modules.cc:285-383); fuse.py
finds them in a memgraph and replaces them by one apply node carrying this descriptor.
"""
from . import _lib

_FIELDS = ("batch", "heads", "rows", "keys", "head_dim", "skip_known", "skip_from")
_STRIDES = ("q_stride", "k_stride", "v_stride", "out_stride")


class attention_t:
    def __init__(self, batch, heads, rows, keys, head_dim, q_stride, k_stride, v_stride, out_stride,
                 mask_stride, skip_known=0, skip_from=0):
        self.batch, self.heads, self.rows, self.keys, self.head_dim = int(batch), int(heads), int(rows), int(keys), int(head_dim)
        self.q_stride = [int(x) for x in q_stride]        # elements: batch, head, row
        self.k_stride = [int(x) for x in k_stride]        # batch, head, key
        self.v_stride = [int(x) for x in v_stride]        # batch, head, key
        self.out_stride = [int(x) for x in out_stride]    # batch, head, row
        self.mask_stride = int(mask_stride)
        self.skip_known, self.skip_from = int(skip_known), int(skip_from)

    @staticmethod
    def from_json(d):
        return attention_t(*[d[f] for f in ("batch", "heads", "rows", "keys", "head_dim")],
                           d["q_stride"], d["k_stride"], d["v_stride"], d["out_stride"], d["mask_stride"],
                           d.get("skip_known", 0), d.get("skip_from", 0))

    def to_json(self):
        d = {f: getattr(self, f) for f in _FIELDS}
        for f in _STRIDES:
            d[f] = list(getattr(self, f))
        d["mask_stride"] = self.mask_stride
        return d

    def eligible(self):
        """What the kernel serves: head dim a multiple of 8 up to 128, strides multiples of 8."""
        if self.head_dim % 8 or self.head_dim > 128 or self.batch > 65535 or self.heads > 65535:
            return False
        return all(x % 8 == 0 for f in _STRIDES for x in getattr(self, f))

    def flops(self):
        return 4 * self.batch * self.heads * self.rows * self.keys * self.head_dim

    def algorithmic_bytes(self):
        bh = self.batch * self.heads
        return 2 * (bh * self.head_dim * (2 * self.rows + 2 * self.keys) + self.rows * self.keys)

    def c_struct(self):
        c = _lib.es_attention_t()
        for f in _FIELDS:
            setattr(c, f, getattr(self, f))
        for f in _STRIDES:
            v = getattr(self, f)
            for i in range(3):
                getattr(c, f)[i] = v[i]
        c.mask_stride = self.mask_stride
        return c
