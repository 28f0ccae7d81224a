#!/usr/bin/env python3
"""Teach an SGLang source tree the ``ep_xpress_b200`` A2A backend.

    python adapters/sglang/integrate.py "$SGLANG_SOURCE" --check      # dry run
    python adapters/sglang/integrate.py "$SGLANG_SOURCE"              # apply
    python adapters/sglang/integrate.py "$SGLANG_SOURCE" --reverse    # take it out again

The reference ships a unified diff for one audited SGLang revision and an applier around
``git apply`` (adapters/sglang/sglang-v0.5.21.patch, adapters/sglang/apply_patch.py). This is an
edit script instead: each edit names a file, an ANCHOR (lines that must occur exactly once) and
the lines to put before or after it. Inserted blocks carry begin/end markers, which makes
"already applied" and "reverse" exact without git, and an anchor that is missing or ambiguous
stops the run before anything is written. Fewer places are touched than by the reference's
diff: the routed experts run on this library's own grouped GEMM, so SGLang's Triton MoE kernels
and its activation kernel stay as they are.

Targets SGLang v0.5.21 (revision ``e00930c5489053f26d86b179cee0d087f846acbb``); when the tree
is a git checkout the revision is verified unless ``--any-revision`` is given. Nothing is
downloaded and nothing outside the listed files is written.
"""

from __future__ import annotations

import argparse
import subprocess
import sys
from dataclasses import dataclass
from pathlib import Path

REVISION = "e00930c5489053f26d86b179cee0d087f846acbb"
BACKEND = "ep_xpress_b200"
BEGIN = "# >>> ep_xpress_b200"
END = "# <<< ep_xpress_b200"


@dataclass(frozen=True)
class Edit:
    path: str            # relative to the source root
    anchor: str          # consecutive lines that occur exactly once in the file
    lines: str           # what to insert (indentation included); markers are added around it
    where: str = "after"  # "before" or "after" the anchor

    def block(self):
        indent = self.lines[: len(self.lines) - len(self.lines.lstrip(" "))]
        body = self.lines if self.lines.endswith("\n") else self.lines + "\n"
        return f"{indent}{BEGIN}\n{body}{indent}{END}\n"


SRT = "python/sglang/srt/"

EDITS = (
    # -- the backend's name ------------------------------------------------------------------
    Edit(SRT + "layers/moe/utils.py",
         'class MoeA2ABackend(Enum):\n    NONE = "none"\n',
         '    EP_XPRESS_B200 = "ep_xpress_b200"\n'),
    Edit(SRT + "layers/moe/utils.py",
         "    def is_none(self):\n        return self == MoeA2ABackend.NONE\n",
         "    def is_ep_xpress_b200(self):\n        return self == MoeA2ABackend.EP_XPRESS_B200\n\n",
         where="before"),
    # combine happens inside the token dispatcher, as for the DeepEP family
    Edit(SRT + "layers/moe/utils.py",
         "        b.is_deepep()\n        or b.is_deepep_v2()\n",
         "        b.is_ep_xpress_b200()\n        or\n",
         where="before"),
    Edit(SRT + "arg_groups/fields/exec_.py",
         '    moe_a2a_backend: A[\n        Literal[\n            "none",\n',
         '            "ep_xpress_b200",\n'),
    Edit(SRT + "arg_groups/fields/exec_.py",
         '            help="Choose the backend for MoE A2A.",\n            choices=[\n                "none",\n',
         '                "ep_xpress_b200",\n'),
    # expert parallelism spans the TP group
    Edit(SRT + "arg_groups/overrides.py",
         "_A2A_EP_SPANNING_BACKENDS = frozenset(\n    {\n",
         '        "ep_xpress_b200",\n'),
    # -- guards and graph policy, once per server start ----------------------------------------
    Edit(SRT + "arg_groups/moe_hook.py",
         "    a2a_backend = resolved_view(server_args).moe_a2a_backend\n",
         '    if a2a_backend == "ep_xpress_b200":\n'
         "        import os\n"
         "\n"
         "        from ep_xpress_b200.adapters.guards import validate_serving_args\n"
         "\n"
         "        validate_serving_args(resolved_view(server_args), model_config_of(server_args).hf_config)\n"
         '        graph_config = cfg.cuda_graph_config\n'
         '        if os.environ.get("EPX_CUDA_GRAPH", "0") == "1":\n'
         "            if graph_config.decode.backend not in (Backend.FULL, Backend.DISABLED):\n"
         '                raise ValueError("ep_xpress_b200 supports full decode CUDA graphs only")\n'
         "        else:\n"
         "            graph_config = with_phase(graph_config, Phase.DECODE, backend=Backend.DISABLED)\n"
         "        graph_config = with_phase(graph_config, Phase.PREFILL, backend=Backend.DISABLED)\n"
         '        declare_resolution(server_args, "_handle_a2a_moe", cuda_graph_config=graph_config)\n'),
    # -- the dispatcher of every MoE layer -------------------------------------------------------
    Edit(SRT + "layers/moe/fused_moe_triton/layer.py",
         ") -> BaseDispatcher:\n    a2a_backend = get_moe_a2a_backend()\n",
         "    if a2a_backend.is_ep_xpress_b200():\n"
         "        from ep_xpress_b200.adapters.sglang import B200EPDispatcher\n"
         "\n"
         "        if not isinstance(quant_method, UnquantizedFusedMoEMethod):\n"
         '            raise ValueError("ep_xpress_b200 serves unquantized BF16 experts only")\n'
         "        return B200EPDispatcher(moe_runner_config)\n"),
    Edit(SRT + "layers/moe/fused_moe_triton/layer.py",
         "        self.intermediate_size_per_partition = intermediate_size // self.moe_tp_size\n",
         "        if get_moe_a2a_backend().is_ep_xpress_b200() and reduce_results:\n"
         '            raise ValueError("ep_xpress_b200 combines inside its dispatcher; reduce_results must be False")\n'),
    # -- the expert runner ------------------------------------------------------------------------
    Edit(SRT + "layers/moe/moe_runner/triton.py",
         '@register_fused_func("none", "triton")\n',
         '@register_fused_func("ep_xpress_b200", "triton")\n'
         "def fused_experts_ep_xpress_b200(dispatch_output, quant_info, runner_config):\n"
         "    from ep_xpress_b200.adapters.sglang import run_experts\n"
         "\n"
         "    return run_experts(dispatch_output, quant_info, runner_config)\n"
         "\n"
         "\n",
         where="before"),
    # -- full decode graphs: hooks outside capture and before every replay -------------------------
    Edit(SRT + "model_executor/runner_backend/full_cuda_graph_backend.py",
         "        reuse_output_buffer: bool = False,\n    ) -> None:\n",
         "        from sglang.srt.layers.moe.utils import get_moe_a2a_backend\n"
         "\n"
         "        self._ep_xpress_b200 = get_moe_a2a_backend().is_ep_xpress_b200()\n"),
    Edit(SRT + "model_executor/runner_backend/full_cuda_graph_backend.py",
         "        graph = torch.cuda.CUDAGraph()\n",
         "        if self._ep_xpress_b200:\n"
         "            from ep_xpress_b200.adapters.sglang import prepare_graph_capture\n"
         "\n"
         "            prepare_graph_capture()\n",
         where="before"),
    Edit(SRT + "model_executor/runner_backend/full_cuda_graph_backend.py",
         "        with graph_pool_replay_scope():\n            self._graphs[shape_key].replay()\n",
         "        if self._ep_xpress_b200:\n"
         "            from ep_xpress_b200.adapters.sglang import prepare_graph_replay\n"
         "\n"
         "            prepare_graph_replay()\n",
         where="before"),
    # every EP rank must pick the same graph bucket: capacity and launch width derive from it
    Edit(SRT + "utils/common.py",
         "        elif moe_a2a_backend.is_none():\n            return True\n",
         "        elif moe_a2a_backend.is_ep_xpress_b200():\n            return True\n"),
)


class IntegrationError(Exception):
    pass


def strip_blocks(text):
    """The text without any marked block (what `--reverse` writes)."""
    kept, inside = [], False
    for line in text.splitlines(keepends=True):
        mark = line.strip()
        if mark == BEGIN:
            if inside:
                raise IntegrationError("nested begin marker")
            inside = True
        elif mark == END:
            if not inside:
                raise IntegrationError("end marker without a begin marker")
            inside = False
        elif not inside:
            kept.append(line)
    if inside:
        raise IntegrationError("begin marker without an end marker")
    return "".join(kept)


def apply_edits(text, edits, path="<text>"):
    """`text` (without marked blocks) with every edit of one file applied."""
    for edit in edits:
        found = text.count(edit.anchor)
        if found != 1:
            raise IntegrationError(f"{path}: anchor occurs {found} times, expected once:\n{edit.anchor}")
        at = text.index(edit.anchor)
        if edit.where == "after":
            at += len(edit.anchor)
        elif edit.where != "before":
            raise IntegrationError(f"{path}: unknown position {edit.where!r}")
        text = text[:at] + edit.block() + text[at:]
    return text


def plan(source, edits=EDITS, reverse=False):
    """{path: (old text, new text)} for every target file; raises before anything is written."""
    by_file = {}
    for edit in edits:
        by_file.setdefault(edit.path, []).append(edit)
    result = {}
    for relative, file_edits in by_file.items():
        path = Path(source) / relative
        if not path.is_file():
            raise IntegrationError(f"{relative}: not found under {source}")
        old = path.read_text()
        clean = strip_blocks(old)
        new = clean if reverse else apply_edits(clean, file_edits, relative)
        if not reverse:
            compile(new, relative, "exec")          # a syntax error here is a bug of the edit list
        result[relative] = (old, new)
    return result


def git_revision(source):
    try:
        done = subprocess.run(["git", "-C", str(source), "rev-parse", "HEAD"], text=True, capture_output=True)
    except OSError:
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("source", type=Path, help="root of the SGLang source tree (the folder that holds python/)")
    parser.add_argument("--check", action="store_true", help="verify every anchor, write nothing")
    parser.add_argument("--reverse", action="store_true", help="remove the integration")
    parser.add_argument("--any-revision", action="store_true", help="do not insist on the audited revision")
    args = parser.parse_args(argv)
    source = args.source.resolve()
    revision = git_revision(source)
    if revision is not None and revision != REVISION and not args.any_revision:
        raise SystemExit(f"this is SGLang revision {revision}; the edit list was written for {REVISION} "
                         "(--any-revision to try anyway: every anchor is still verified)")
    try:
        changes = plan(source, reverse=args.reverse)
    except IntegrationError as error:
        raise SystemExit(f"nothing was written: {error}")
    pending = {path: new for path, (old, new) in changes.items() if old != new}
    verb = "remove" if args.reverse else "apply"
    if not pending:
        print(f"nothing to {verb}: the tree is already in that state")
        return 0
    if args.check:
        print(f"would {verb} the {BACKEND} integration in {len(pending)} file(s):")
    for path in sorted(pending):
        if not args.check:
            (source / path).write_text(pending[path])
        print(f"  {path}")
    if not args.check:
        print(f"{verb}d; install this library and the SGLang tree into the same environment" if not args.reverse
              else "removed")
    return 0


if __name__ == "__main__":
    sys.exit(main())
