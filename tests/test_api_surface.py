"""Everything public in the reference's `src` package exists under the same import path here, with call
signatures a reference caller can use unchanged: every reference parameter is accepted, by the same name and in
the same position; parameters this framework adds have defaults.  The reference is read as text (ast) from
baseline/_ref, never imported; the test is skipped where it is not installed."""
import ast
import importlib
import inspect
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "train.py").exists(), reason="reference not installed under baseline/_ref")

# Deliberate differences, each with its reason.
DIFFERENT = {
    # the reference's constructor takes (cfg, experts, router) but its own caller passes four arguments
    # (src/model/feed_fwd.py:142), so the 3-argument form never ran; ours takes what the caller passes
    ("src.model.cuda_backend", "CUDAMoEBackend", "__init__"),
}


def _reference_modules():
    for path in sorted(REF.rglob("*.py")):
        rel = path.relative_to(REF).with_suffix("")
        if rel.name == "__init__" or "dist-info" in str(rel):
            continue
        yield "src." + ".".join(rel.parts), path


def _params(args: ast.arguments):
    names = [a.arg for a in args.posonlyargs + args.args]
    return [n for n in names if n not in ("self", "cls")], [a.arg for a in args.kwonlyargs]


def _check_callable(where, ref_args: ast.arguments, ours):
    try:
        sig = inspect.signature(ours)
    except (TypeError, ValueError):
        return []  # a builtin / extension callable: nothing to compare
    positional, kwonly = _params(ref_args)
    mine = [p for p in sig.parameters.values() if p.name not in ("self", "cls")]
    if any(p.kind is p.VAR_POSITIONAL for p in mine) and any(p.kind is p.VAR_KEYWORD for p in mine):
        return []  # forwards everything
    problems = []
    mine_pos = [p for p in mine if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    for i, name in enumerate(positional):
        if i >= len(mine_pos) or mine_pos[i].name != name:
            got = mine_pos[i].name if i < len(mine_pos) else "nothing"
            problems.append(f"{where}: parameter {i} is `{name}` in the reference, `{got}` here")
            break
    for extra in mine_pos[len(positional):]:
        if extra.default is inspect.Parameter.empty:
            problems.append(f"{where}: added parameter `{extra.name}` has no default")
    names = {p.name for p in mine}
    for name in kwonly:
        if name not in names and not any(p.kind is p.VAR_KEYWORD for p in mine):
            problems.append(f"{where}: keyword `{name}` is missing")
    return problems


def test_reference_import_paths_names_and_signatures():
    problems = []
    checked = 0
    for module_name, path in _reference_modules():
        tree = ast.parse(path.read_text())
        try:
            module = importlib.import_module(module_name)
        except Exception as exc:  # noqa: BLE001
            problems.append(f"{module_name}: cannot be imported here ({type(exc).__name__}: {exc})")
            continue
        for node in tree.body:
            if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and not node.name.startswith("_"):
                if not hasattr(module, node.name):
                    problems.append(f"{module_name}.{node.name}: missing")
                    continue
                ours = getattr(module, node.name)
                checked += 1
                if isinstance(node, ast.FunctionDef):
                    problems += _check_callable(f"{module_name}.{node.name}", node.args, ours)
                    continue
                is_autograd_fn = any("Function" in ast.unparse(b) for b in node.bases)
                for item in node.body:
                    if not isinstance(item, ast.FunctionDef) or (item.name.startswith("_") and item.name != "__init__"):
                        continue
                    if any("validator" in ast.unparse(d) for d in item.decorator_list):
                        continue  # pydantic hooks: run by the schema, not called by users
                    if is_autograd_fn:  # used as Name.apply(*forward's arguments after ctx)
                        if item.name == "forward":
                            item.args.args = [a for a in item.args.args if a.arg != "ctx"]
                            problems += _check_callable(f"{module_name}.{node.name}.apply", item.args, ours.apply)
                        continue
                    if (module_name, node.name, item.name) in DIFFERENT:
                        continue
                    if not hasattr(ours, item.name):
                        problems.append(f"{module_name}.{node.name}.{item.name}: missing")
                        continue
                    problems += _check_callable(f"{module_name}.{node.name}.{item.name}", item.args, getattr(ours, item.name))
    assert checked > 40, "the reference tree was not found where expected"
    assert not problems, "\n".join(problems)


def test_extension_has_the_reference_entry_points():
    from nanotitan_b200.ops.ext import get_ext, have_ext

    if not have_ext():
        pytest.skip("the extension is not built")
    ext = get_ext()
    for name in ("random_op", "copy_scalar", "copy_vector", "count_expert_kernel", "pack_tokens_kernel", "combine_tokens_kernel",
                 "combine_kernel_backward", "gemm_kernel", "tiled_gemm_kernel", "naive_gemm_kernel", "pack_kernel_backward",
                 "grouped_gemm_kernel", "bwd_grouped_gemm_dW_kernel", "bwd_grouped_gemm_dX_kernel"):
        assert callable(getattr(ext, name, None)), name


def test_function_class_spellings_reach_the_same_operations():
    import torch

    from src.model import moe_ops

    torch.manual_seed(0)
    x = torch.randn(6, 4)
    experts = torch.tensor([[0, 2], [1, 2], [0, 1], [2, 0], [1, 0], [2, 1]], dtype=torch.int32)
    gates = torch.rand(6, 2)
    counts = torch.bincount(experts.flatten().long(), minlength=3)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32)
    a = moe_ops.PackTokensFN.apply(x, gates, experts, offsets.clone())
    b = moe_ops.pack_tokens_fn(x, gates, experts, offsets.clone())
    assert all(torch.equal(p, q) for p, q in zip(a, b))
    px, ptok, pexp, pw = a
    assert torch.equal(px, x[ptok.long()]) and ptok.dtype == torch.int32 and pw.dtype == torch.float32
    w = torch.randn(3, 4, 5)
    assert torch.equal(moe_ops.GroupedGEMM_FN.apply(px, offsets, w), moe_ops.grouped_gemm_fn(px, w, offsets))
    y = moe_ops.CombineTokensFN.apply(px, ptok, pw, 6, 4)
    torch.testing.assert_close(y, x * gates.sum(1, keepdim=True), rtol=1e-5, atol=1e-6)
    with pytest.raises(TypeError):
        moe_ops.PackTokensFN()


def test_type_stub_matches_the_built_extension():
    from nanotitan_b200.ops import ext

    if not ext.have_ext():
        pytest.skip("the extension is not built")
    assert ext.STUB_PATH.read_text() == ext.stub_text(), "run `python -m nanotitan_b200.ops.ext --stub`"
