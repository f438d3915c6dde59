"""Runs in a child process with ONLY the reference project importable (``baseline/_ref`` through the third-party
stand-ins of ``baseline/_stubs``): for every job of the input file it builds the reference model of a family from config
keywords, loads the given parameters, runs ``compute_loss`` and its backward on the given batch and records losses, codes
and gradients (importing the reference takes tens of seconds, so all jobs share one process).
``tests/test_reference_parity.py`` runs the same inputs through this package and compares.

    python reference_side.py <input.pt> <output.pt>
"""

import sys


def main(inp: str, out: str) -> None:
    import torch

    jobs = torch.load(inp, weights_only=False)  # name -> job
    results = {}
    for name, job in jobs.items():
        try:
            results[name] = run_job(job)
        except Exception as e:  # noqa: BLE001  (reported per case by the parent)
            import traceback

            results[name] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"}
    torch.save(results, out)


def run_training(job: dict) -> dict:
    """A few steps of the reference's own ``Trainer.fit`` on the given batches (on the job's device); returns the
    parameters afterwards."""
    import tempfile

    import llamascopium as L
    import torch
    from llamascopium.models.sparse_dictionary import SparseDictionary

    kw = dict(job["config"])
    kw["dtype"] = getattr(torch, kw["dtype"])
    model = SparseDictionary.from_config(getattr(L, job["config_class"])(**kw))
    model.load_state_dict({k: v.to(kw["device"]) for k, v in job["state"].items()}, strict=False)
    model.set_dataset_average_activation_norm(job["norm"])
    batches = [{k: v.to(kw["device"]) for k, v in b.items()} for b in job["batches"]]
    with tempfile.TemporaryDirectory() as tmp:
        tcfg = L.TrainerConfig(exp_result_path=tmp, **job["trainer"])
        L.Trainer(tcfg).fit(model, iter([batches[0]] + batches))  # (the reference consumes one batch while sizing its schedule)
    return {"state": {k: v.detach().cpu() for k, v in model.state_dict().items()}}


def run_job(job: dict) -> dict:
    if job.get("kind") == "train":
        return run_training(job)
    import llamascopium as L
    import torch
    from llamascopium.models.sparse_dictionary import SparseDictionary

    cfg_cls = getattr(L, job["config_class"])
    kw = dict(job["config"])
    kw["dtype"] = getattr(torch, kw["dtype"])
    cfg = cfg_cls(**kw)
    model = SparseDictionary.from_config(cfg) if hasattr(SparseDictionary, "from_config") else None
    if model is None:
        raise SystemExit("the reference has no SparseDictionary.from_config")
    missing = model.load_state_dict(job["state"], strict=False)
    assert not missing.unexpected_keys, missing
    if job.get("norm"):
        model.set_dataset_average_activation_norm(job["norm"])
    batch = model.normalize_activations(dict(job["batch"])) if job.get("normalize", True) else dict(job["batch"])
    dead = {}

    def update_dead(feature_acts, mask, specs):
        fired = feature_acts.reshape(-1, feature_acts.shape[-1]).sum(0) > 0
        dead["is_dead"] = ~fired
        return dead["is_dead"]

    extra = dict(job.get("loss_kwargs", {}))
    if extra.get("auxk_coefficient", 0.0) > 0.0:
        extra["update_dead_statistics"] = update_dead
    res = model.compute_loss(batch, return_aux_data=True, **extra)
    res["loss"].backward()
    rec = {"loss": res["loss"].detach(), "feature_acts": res["feature_acts"].detach(), "reconstructed": res["reconstructed"].detach(),
           "grads": {n: p.grad.detach() for n, p in model.named_parameters() if p.grad is not None}}  # fmt: skip
    for key in ("l_rec", "l_s", "l_p", "l_aux"):
        if res.get(key) is not None:
            rec[key] = res[key].detach()
    return rec


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
