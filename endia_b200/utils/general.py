"""Graph walks of the autograd engine (endia/utils/general.mojo:18-62), iterative so that deep
graphs do not hit the interpreter's recursion limit."""


def top_order(out):
    """Depth-first post-order over `args` starting at `out` (general.mojo:26-32): every node
    appears after all of its arguments."""
    trace, seen = [], set()
    stack = [(out, 0)]
    seen.add(id(out))
    while stack:
        node, i = stack.pop()
        args = node.args_
        if i < len(args):
            stack.append((node, i + 1))
            a = args[i]
            if id(a) not in seen:
                seen.add(id(a))
                stack.append((a, 0))
        else:
            node.id = len(trace)
            trace.append(node)
    return trace


def reset_node_id_recursive(out):
    for node in top_order(out):
        node.id = -1


def remove_grad_rec(out):
    """Drop the stored gradient of every node reachable from `out` (general.mojo:59-62)."""
    for node in top_order(out):
        node.remove_grad()
        node.id = -1


def zero_grad_rec(out):
    """general.mojo:44-47; like the reference this removes the gradients."""
    remove_grad_rec(out)


class HostBatchFeeder:
    """Feeds host batches to the device through two sets of device arrays and a copy stream: while
    a step computes on one set, the next batch is copied into the other. `host` is a list of pinned
    torch tensors (one per input); next() returns the list of device Arrays holding the batch it
    was last asked to stage and starts staging the following one."""

    def __init__(self, host, shapes):
        import torch
        from .._array import Array, device
        self._torch = torch
        self.host = host
        self.sets = [[Array(list(s)) for s in shapes] for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=device())
        self.ready = [None, None]
        self.last_use = [None, None]
        self.cur = 0

    def _stage(self, idx):
        torch = self._torch
        if self.last_use[idx] is not None:
            self.copy_stream.wait_event(self.last_use[idx])   # the set's last readers are done
        with torch.cuda.stream(self.copy_stream):
            for arr, h in zip(self.sets[idx], self.host):
                arr.buf[:h.numel()].copy_(h.reshape(-1), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self.ready[idx] = ev

    def next(self):
        torch = self._torch
        # everything enqueued so far includes all readers of the set handed out last time
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.last_use[self.cur ^ 1] = ev
        if self.ready[self.cur] is None:
            self._stage(self.cur)
        torch.cuda.current_stream().wait_event(self.ready[self.cur])
        self.ready[self.cur] = None
        out = self.sets[self.cur]
        self.cur ^= 1
        return out

    def prefetch(self):
        """Start the copy of the following batch (call after the step's kernels are enqueued)."""
        if self.ready[self.cur] is None:
            self._stage(self.cur)


class CapturedStep:
    """Replays a step as one CUDA graph. `fn()` must be static: the same ops on the same shapes
    every call, inputs read from Arrays that exist before the capture (refill them in place, e.g.
    with HostBatchFeeder-style copies, between replays), no host reads inside (to_numpy, item).
    fn runs `warmup` times eagerly first, so that first-use set-up (kernel attributes, twiddle
    tables) is done, then once more under capture; its return value from that run is kept and
    returned by every call, its Arrays refilled by the replay. A step whose kernels are short next
    to the ~25 us of host work per launch (the create_graph=True double-backward step has about
    85 launches) becomes GPU-bound this way."""

    def __init__(self, fn, warmup=2, optimizers=()):
        """`optimizers`: the optimizers whose step() runs inside fn. Their step count changes from
        step to step, so it moves to the device for the capture (begin_capture / end_capture) and
        the host copy is advanced after every replay (after_replay)."""
        import torch
        from .._array import device
        device()
        self.optimizers = list(optimizers)
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        from .. import _lib
        for opt in self.optimizers:
            opt.begin_capture()
        torch.cuda.synchronize()
        before = _lib.lib.endia_b200_launch_count()
        self.graph = torch.cuda.CUDAGraph()
        from ..autograd import state as _state
        from .._array import drop_operand_parts
        _state.capture_parts = []      # leaves whose GEMM operand parts are shared inside this step
        try:
            with torch.cuda.graph(self.graph):
                self.out = fn()
        except BaseException:
            for opt in self.optimizers:
                opt.end_capture()
            raise
        finally:
            for leaf in _state.capture_parts:
                drop_operand_parts(leaf)
            _state.capture_parts = None
        torch.cuda.synchronize()
        # kernels of this library inside the graph (endia_b200_launch_count only sees enqueues)
        self.launches_per_replay = int(_lib.lib.endia_b200_launch_count() - before)
        self.replays = 0

    def __call__(self):
        self.graph.replay()
        self.replays += 1
        for opt in self.optimizers:
            opt.after_replay()
        return self.out

    def release(self):
        """Back to op-by-op steps: the optimizers count on the host again."""
        for opt in self.optimizers:
            opt.end_capture()
        self.optimizers = []
