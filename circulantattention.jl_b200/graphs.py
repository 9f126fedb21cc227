"""CUDA-graph capture of calls into the library.

Every entry point of the C ABI orders its work on the stream it is given, allocates nothing itself, never
synchronises the device, and joins the helper stream of `ca_attention_bwd` back by events, so a forward and its
backward can be recorded once into a CUDA graph and replayed: a replay costs the host one launch instead of the
Python and autograd work of the step.  The tensors the captured function reads are the graph's static inputs:
write new values INTO them (`copy_`) before a replay; the tensors it produced (outputs, `.grad` of the leaves) are
overwritten by every replay.
"""
import torch


def capture(fn, stream=None, warmup=2):
    """Runs `fn()` `warmup` times eagerly on a side stream (so that every lazily created buffer, tensor map and
    helper stream exists), then once more under capture.  Returns `(graph, result_of_fn)`; `graph.replay()`
    repeats the recorded work on the current stream.

    For a training step, clear the leaves' gradients first (`x.grad = None`) so that the backward recorded in
    the graph writes fresh `.grad` tensors from the graph's own memory pool, as
    https://pytorch.org/docs/stable/notes/cuda.html#whole-network-example does."""
    side = stream if stream is not None else torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    # thread_local: other host threads (a process group's watchdog, a data loader) may keep calling the CUDA
    # runtime while this thread records
    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
        result = fn()
    return graph, result
