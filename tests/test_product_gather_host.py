"""Host logic of `transformer.product_gather` on CPU: which of the three routes a sharded product takes (nodes handed to
the gather kernel, a finished slice through the exchange, or the process group), with the device calls replaced by
recording stand-ins. The device side of the same routes is `tests/test_gpu_exchange.py` and `tests/test_gpu_multi.py`."""
import pytest
import torch

from mojolearn_b200 import transformer


class _Lin(object):
    def __init__(self, n, k, bias=False):
        self.w, self.scale, self.kind = torch.zeros((n, k)), None, 0
        self.bias = torch.zeros((n,)) if bias else None
        self.out_features, self.in_features = n, k


class _Exchange(object):
    def __init__(self, fits=True):
        self.fits, self.calls = fits, []

    def takes_shape(self, m, w):
        self.calls.append(("takes_shape", m, w))
        return self.fits

    def takes(self, part):
        return self.fits

    def gather(self, part):
        self.calls.append(("gather", tuple(part.shape)))
        return part.repeat(1, 2)

    def gather_nodes(self, ws, nodes, m, n, bias, act):
        self.calls.append(("gather_nodes", nodes, m, n, bias is not None, act))
        return torch.zeros((m, 2 * (n // 2 if act >= 4 else n)))


@pytest.fixture
def ops(monkeypatch):
    log = []

    def product_nodes(a, b, bscale=None, wkind=0, bias=None, act=0):
        log.append(("product_nodes", act))
        n = b.shape[0]
        if product_nodes.nodes > 1:
            return None, torch.zeros((16,)), product_nodes.nodes
        return torch.zeros((a.shape[0], n // 2 if act >= 4 else n)), None, 1

    def product(a, b, bscale=None, wkind=0, op=0, bias=None, act=0, **kw):
        log.append(("product", act))
        n = b.shape[0]
        return torch.zeros((a.shape[0], n // 2 if act >= 4 else n))

    product_nodes.nodes = 16
    monkeypatch.setattr(transformer.torch_ops, "product_nodes", product_nodes)
    monkeypatch.setattr(transformer.torch_ops, "product", product)
    monkeypatch.setattr(transformer, "gather_columns", lambda part, group, exchange: (log.append(("gather_columns", tuple(part.shape))), part)[1])
    return log, product_nodes


def test_split_product_hands_its_nodes_to_the_gather(ops):
    log, pn = ops
    ex = _Exchange()
    out = transformer.product_gather(_Lin(256, 2048, bias=True), torch.zeros((32, 2048)), 1, None, ex)
    assert out.shape == (32, 512)
    assert log == [("product_nodes", 1)]
    assert ex.calls == [("takes_shape", 32, 256), ("gather_nodes", 16, 32, 256, True, 1)]


def test_gated_store_halves_the_gathered_width(ops):
    log, pn = ops
    ex = _Exchange()
    out = transformer.product_gather(_Lin(2048, 2048), torch.zeros((32, 2048)), 4, None, ex)
    assert out.shape == (32, 2048)  # two ranks x 1024 activated columns
    assert ex.calls == [("takes_shape", 32, 1024), ("gather_nodes", 16, 32, 2048, False, 4)]


def test_unsplit_product_goes_through_the_plain_gather(ops):
    log, pn = ops
    pn.nodes = 1
    ex = _Exchange()
    out = transformer.product_gather(_Lin(256, 64), torch.zeros((4, 64)), 0, None, ex)
    assert out.shape == (4, 512)
    assert log == [("product_nodes", 0)] and ex.calls[-1] == ("gather", (4, 256))


@pytest.mark.parametrize("case", ["no exchange", "does not fit", "odd width", "loopback without the entry"])
def test_everything_else_takes_the_finished_product(ops, case):
    log, pn = ops
    ex, n = _Exchange(), 256
    if case == "no exchange":
        ex = None
    elif case == "does not fit":
        ex = _Exchange(fits=False)
    elif case == "odd width":
        n = 258  # not a multiple of 4: the fold in the gather kernel owns four cells of one row per thread
    else:
        ex = type("Plain", (), {"takes": lambda self, p: False})()
    transformer.product_gather(_Lin(n, 64), torch.zeros((4, 64)), 0, None, ex)
    assert log == [("product", 0), ("gather_columns", (4, n))]
