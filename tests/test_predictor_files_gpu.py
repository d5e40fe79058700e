"""PredictorBase.load_model: the reference's predictor directory format, one `<src>-<dst>.pt` file per
(source index, predicted layer) pair of the prediction window (src/cpp_worker/predictor.cpp:608-636).
The files hold a state dict or a TorchScript module of one MLP hidden -> d -> num_expert; loaded
predictors must drive the same prefetches as the oracle computing with the same weights."""
import numpy as np
import pytest
import torch

from oracle import moe_math as om
from oracle import srs_policy as sp
from promoe_b200 import cpp_worker as cw
from tests.helpers import TinyModel, dev_bf16

pytestmark = pytest.mark.gpu


class Mlp(torch.nn.Module):
    def __init__(self, H, D, E):
        super().__init__()
        self.fc1, self.fc2 = torch.nn.Linear(H, D), torch.nn.Linear(D, E)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


def test_load_model_directory_and_predict(lib, tmp_path):
    model = TinyModel(seed=6, L=4, E=12, H=128, I=64, k=3)
    torch.manual_seed(0)
    pairs = [(0, 0), (1, 1), (1, 2), (1, 3)]           # default window of a four-layer stack
    nets = {}
    for i, (src, dst) in enumerate(pairs):
        net = Mlp(model.H, 32, model.E)
        with torch.no_grad():
            for p in net.parameters():                  # bf16-representable matrices: both sides compute on the same values
                if p.dim() == 2:
                    p.copy_((p * 3.0).to(torch.bfloat16).float())
        nets[(src, dst)] = net
        path = tmp_path / f"{src}-{dst}.pt"
        if i % 2 == 0:
            torch.save(net.state_dict(), path)          # a plain state dict
        else:
            torch.jit.script(net).save(str(path))       # a TorchScript module, as the reference loads
    meta = cw.ModuleMeta(model.L, model.E)
    meta.init_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
    meta.init_from_map({"cache_rate": "0.5", "num_expert_per_token": str(model.k), "num_predict_expert_per_layer": "3",
                        "predictor_model_path": str(tmp_path), "predict_from_moe_input": "true"})
    loader = cw.ModelLoader(meta)
    for l in range(model.L):
        for e in range(model.E):
            for n, w in zip(("gate_proj.weight", "up_proj.weight", "down_proj.weight"), model.experts[l][e]):
                loader.add_one_expert_param(torch.from_numpy(w), l, e, n)
    predictor = cw.PredictorBase.create(meta)
    mngr = cw.PrefetchMngr(meta, loader, predictor)
    mngr.init_gpu_mem_buffer()
    predictor.load_model()
    assert sorted(predictor.loaded) == pairs
    cache = meta.cache
    for l in range(model.L):
        cache.set_layer_weights(l, dev_bf16(model.gate_w[l]), model.I, model.k, False,
                                gate_bias=torch.from_numpy(model.gate_bias[l]).cuda())
    cache.enable_event_log(True)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=0.5, num_predict=3)
    for x in model.hidden_stream(4, 4):
        xd = dev_bf16(x)
        for l in range(model.L):
            for (src, dst), net in sorted(nets.items()):
                if src == l:
                    sd = {k: v.detach().numpy() for k, v in net.state_dict().items()}
                    scores = om.predictor_scores(x, sd["fc1.weight"], sd["fc1.bias"], sd["fc2.weight"], sd["fc2.bias"])
                    oc.prefetch_layer(dst, om.rank_experts(scores, oc.num_predict))
            cache.forward(l, xd)
            ref_ids, _ = model.canonical_routing(l, x)
            oc.report_layer(l, om.unique_sorted_experts(ref_ids))
    torch.cuda.synchronize()
    assert cache.events() == oc.events
    assert cache.stats()["prefetch_miss"] > 0
    with pytest.raises(FileNotFoundError):
        predictor.load_model(str(tmp_path / "missing"))
    cache.close()
