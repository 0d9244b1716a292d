"""Child process of the gated_deltanet GPU parity test: the FLA library's model (its Triton kernels) and the
native model on the same weights; prints both losses as JSON.  Runs apart from the test process so that a
failure inside the library's kernels cannot leave that process with a broken CUDA context."""
import json
import os
import sys
import warnings

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch


def main():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from fla.models import GatedDeltaNetConfig as FC, GatedDeltaNetForCausalLM as FM
    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.ops import _cuda

    torch.manual_seed(0)
    cfg = dict(vocab_size=256, hidden_size=256, num_hidden_layers=2, num_heads=2, num_v_heads=4, head_dim=128, expand_v=1.0, hidden_ratio=4)
    lib = FM(FC(**cfg, fuse_norm=False, fuse_swiglu=False, fuse_cross_entropy=False)).to("cuda", torch.bfloat16).eval()
    mine = create_model_from_config("gated_deltanet", cfg).to("cuda", torch.bfloat16).eval()
    mine.load_state_dict(mine.convert_hf_state_dict(lib.state_dict()), strict=True)
    ids = torch.randint(0, 256, (1, 300), device="cuda")
    n0 = _cuda.launch_count
    with torch.no_grad():
        got = mine(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids)["loss"]
        torch.cuda.synchronize()
        native_launches = _cuda.launch_count - n0
        want = lib(input_ids=ids, labels=ids).loss
    torch.cuda.synchronize()
    print(json.dumps({"native": float(got), "library": float(want), "native_launches": native_launches}))


if __name__ == "__main__":
    main()
