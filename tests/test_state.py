"""OptimizerModule and the state-dict helpers."""

import copy

import pytest
import torch

from optimizers_b200.utils.state import OptimizerModule, extract_state_dict_content, update_param_state_dict_object


class Leaf(OptimizerModule):
    def __init__(self):
        self.w = torch.arange(3.0)
        self.flag = True


class Tree(OptimizerModule):
    def __init__(self):
        self.t = torch.ones(2)
        self.pair = (torch.zeros(2), torch.full((2,), 5.0))
        self.names = ("a", "b")
        self.leaf = Leaf()
        self.table = {"x": torch.tensor([1.0]), "empty": {}}
        self.count = 3


def test_state_dict_layout():
    sd = Tree().state_dict()
    assert set(sd) == {"t", "pair", "leaf", "table"}  # non-tensors and empty containers dropped
    assert set(sd["pair"]) == {0, 1} and set(sd["leaf"]) == {"w"} and set(sd["table"]) == {"x"}
    sd_all = Tree().state_dict(store_non_tensors=True)
    assert sd_all["count"] == 3 and sd_all["names"] == {0: "a", 1: "b"} and sd_all["leaf"]["flag"] is True


def test_load_is_in_place_and_repairs_string_keys():
    tree = Tree()
    views = (tree.t, tree.pair[1], tree.leaf.w)
    sd = copy.deepcopy(tree.state_dict())
    sd["t"] += 1
    sd["pair"] = {"0": sd["pair"][0] + 2, "1": sd["pair"][1] + 3}  # keys as a flattened checkpoint returns them
    sd["leaf"]["w"] *= 2
    tree.load_state_dict(sd)
    assert tree.t is views[0] and tree.pair[1] is views[1] and tree.leaf.w is views[2]
    assert torch.equal(tree.t, torch.full((2,), 2.0)) and torch.equal(tree.pair[1], torch.full((2,), 8.0))
    assert torch.equal(tree.leaf.w, torch.tensor([0.0, 2.0, 4.0])) and tree.count == 3
    with pytest.raises(KeyError):
        tree.load_state_dict({"pair": {"0": torch.zeros(2)}})


def test_update_and_extract_helpers():
    tree = Tree()
    live = {"blk": {"mod": tree, "buf": torch.zeros(2)}, "step": torch.tensor(1)}
    flat = extract_state_dict_content(live)
    assert isinstance(flat["blk"]["mod"], dict) and flat["blk"]["buf"] is live["blk"]["buf"]
    incoming = copy.deepcopy(flat)
    incoming["blk"]["buf"] += 7
    incoming["step"] = torch.tensor(9)
    incoming["blk"]["mod"]["t"] += 4
    update_param_state_dict_object(live, incoming)
    assert live["step"].item() == 9 and torch.equal(live["blk"]["buf"], torch.full((2,), 7.0))
    assert torch.equal(tree.t, torch.full((2,), 5.0))
    with pytest.raises(KeyError):
        update_param_state_dict_object(live, {"blk": incoming["blk"]})
    update_param_state_dict_object(live, {"blk": incoming["blk"]}, enable_missing_key_check=False)
