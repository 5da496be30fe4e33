"""Eager stand-ins for the reference's graph tracer, for scripts that wrap their forward pass in it
(examples/llama3.py:360-367: ``trace_function`` -> ``TraceGraphExecutor(...).execute`` and ``dump_graphviz(...).save``).

The reference records the operators a function dispatches into a graph (minit/trace/function.py:14-34) and replays the
graph (minit/trace/executor.py:49-159).  Nothing is recorded here: ``trace_function`` keeps the function and the shapes
and dtypes of the example arguments, the executor calls the function.  Replaying a fixed launch sequence is what CUDA
graphs are for in this package (the decoder layer and the bench capture theirs); a tracing compiler is not rebuilt."""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

from .tensor import Tensor, to_immediate_shape


class EagerGraph:
    """What ``trace_function`` returns: the function and the signature it was shown."""

    def __init__(self, function: Callable, args: Sequence) -> None:
        self.function = function
        self.inputs: List[Tuple[Tuple[int, ...], str]] = [
            (to_immediate_shape(arg.shape), arg.dtype) if isinstance(arg, Tensor) else ((), type(arg).__name__) for arg in args]


def trace_function(function: Callable, args: Sequence) -> EagerGraph:
    return EagerGraph(function, args)


class TraceGraphExecutor:
    def __init__(self, graph: EagerGraph) -> None:
        self.graph = graph

    def execute(self, *args) -> tuple:
        outputs = self.graph.function(*args)
        if outputs is None:
            return ()
        return tuple(outputs) if isinstance(outputs, (tuple, list)) else (outputs,)

    __call__ = execute


class _Dot:
    def __init__(self, text: str) -> None:
        self.source = text

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.source)


def dump_graphviz(graph: EagerGraph) -> _Dot:
    """One node for the function, one per input: the operators inside it are not recorded."""
    name = getattr(graph.function, "__name__", "function")
    lines = ["digraph G {", f'  f [shape=box, label="{name} (eager)"];']
    for i, (shape, dtype) in enumerate(graph.inputs):
        lines.append(f'  in{i} [label="{dtype}{list(shape)}"];')
        lines.append(f"  in{i} -> f;")
    lines.append("}")
    return _Dot("\n".join(lines) + "\n")
