"""Two gloo ranks train the tiny configuration; the last rank raises inside its third step.  The other
rank must stop with ``PeerFailure`` (learned from the store between steps) instead of waiting in a
collective, and the script reports how each rank ended."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    out = sys.argv[1]
    rank = int(os.environ["RANK"])
    from tiny_run import make_config

    from lmms_engine_b200.launch.cli import create_train_task
    from lmms_engine_b200.utils.failure import PeerFailure

    cfg = make_config(out, "native", steps=8, extra_args={"heartbeat_timeout": 5.0, "ddp_timeout": 20})
    runner = create_train_task(cfg).build()
    trainer = runner.trainer
    if rank == int(os.environ["WORLD_SIZE"]) - 1:
        orig = trainer.training_step
        calls = {"n": 0}

        def flaky(batch, do_step):
            calls["n"] += 1
            if calls["n"] == 3:
                raise ValueError("injected host-side failure")
            return orig(batch, do_step)

        trainer.training_step = flaky
    how = "finished"
    try:
        runner.run()
    except PeerFailure as e:
        how = f"peer_failure: {e}"
    except ValueError as e:
        how = f"raised: {e}"
    except RuntimeError as e:  # a collective that timed out because the peer left
        how = f"runtime_error: {str(e)[:120]}"
    with open(os.path.join(out, f"end_rank{rank}.json"), "w") as f:
        json.dump({"how": how, "step": trainer.global_step}, f)
    os._exit(0)  # skip process-group teardown: the peer is gone


if __name__ == "__main__":
    main()
