import torch


def cos_sim(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max())


def assert_close(got, want, cos=0.999, rel=None, name=""):
    c = cos_sim(got, want)
    assert c > cos, f"{name}: cosine {c} <= {cos}"
    if rel is not None:
        err = max_abs(got, want) / (float(want.double().abs().max()) + 1e-30)
        assert err < rel, f"{name}: max rel err {err} >= {rel}"
