"""CPU: the tree operations of nn.Module (state_dict paths, parameter order, train / eval, load_state_dict and its
error texts) on tensors that need no GPU.  The contract is the reference's (gradtuity/nn.py:34-158; its tests
match on "missing" and "unexpected": gradtuity/tests/test_nn.py)."""
import pytest

from gradtuity_b200.nn import Module
from gradtuity_b200.tensor import Storage, Tensor


def _t(shape, requires_grad=True):
    return Tensor._wrap(Storage(0, 4, owns=False), shape, requires_grad=requires_grad)


class Leaf(Module):
    def __init__(self):
        super().__init__()
        self.weight = _t((2, 3))
        self.bias = _t((3,))
        self.frozen = _t((3,), requires_grad=False)


class Top(Module):
    def __init__(self):
        super().__init__()
        self.layers = [Leaf(), Leaf()]
        self.head = Leaf()
        self.note = "not a parameter"


def test_paths_order_and_modes():
    m = Top()
    assert sorted(m.state_dict()) == ["head.bias", "head.weight", "layers.0.bias", "layers.0.weight", "layers.1.bias", "layers.1.weight"]
    assert m.parameters() == [m.state_dict()[k] for k in sorted(m.state_dict())] and len(m.parameters()) == 6
    assert m.eval() is m and not m.training and not m.layers[1].training and not m.head.training
    m.train()
    assert m.training and m.layers[0].training and m.head.training


def test_load_state_dict_replaces_tensors_and_reports_key_errors():
    m = Top()
    new = _t((2, 3))
    state = dict(m.state_dict())
    state["layers.1.weight"] = new
    m.load_state_dict(state)
    assert m.layers[1].weight is new and m.layers[0].weight is state["layers.0.weight"]
    with pytest.raises(ValueError, match="missing"):
        m.load_state_dict({"head.weight": new})
    with pytest.raises(ValueError, match="unexpected"):
        m.load_state_dict(dict(state, nowhere=new))
    m.load_state_dict({"head.weight": new, "nowhere": new}, strict=False)
    assert m.head.weight is new
