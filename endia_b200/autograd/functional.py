"""Reverse-mode autodiff: backward/jacrev, imperative grad, and the functional transforms
grad / jacobian / hessian / value_and_grad (endia/autograd/functional.mojo:21-243 and the eager
branch of Callable.__call__, endia/compile/callable.mojo:100-197). The walk only enqueues kernels;
nothing synchronises with the device."""
from . import state as _state
from ..utils.general import top_order, reset_node_id_recursive, remove_grad_rec


def backward(arg, create_graph=False):
    jacrev(arg, create_graph)


def jacrev(arg, create_graph=False, only_for=None):
    """Reverse walk over the graph of `arg` (autograd/functional.mojo:26-67).

    `only_for` (a list of Arrays, used by the imperative grad(outs, inputs)): VJPs are evaluated
    only along the paths from `arg` to these arrays; gradients that cannot reach one of them (e.g.
    the weight gradients when only the input gradient of a network is asked for) are not computed.
    The gradients of the listed arrays are the same either way.

    A 1-D, one-element output is seeded with ones(1); any other output gets an identity seed of
    shape out.shape + out.shape, so the stored gradients are full Jacobians (:34-38). Gradients
    ACCUMULATE into nodes that already hold one (:55-57). Unless `create_graph`, the graph edges of
    each new gradient are cut (:63-65)."""
    from ..functional.init_ops import ones, eye
    from ..functional.view_ops import reshape
    from ..functional.binary_ops import add
    out = arg
    trace = top_order(out)
    wanted = None
    if only_for is not None:
        # nodes whose value depends on one of the listed arrays (every node comes after its arguments)
        targets = {id(a) for a in only_for}
        wanted = set()
        for node in trace:
            if id(node) in targets or any(id(a) in wanted for a in node.args_):
                wanted.add(id(node))
    last_dim = out.shape()[-1]
    if out.ndim() != 1 or last_dim != 1:
        seed = reshape(eye(out.size()), out.shape() + out.shape())
    else:
        seed = ones([last_dim])
        seed._is_ones_seed = True   # lets a fused VJP skip the multiplication by one
    out.grad_(seed)
    # Number of graph edges into every node, so that a leaf's hook fires once its last
    # contribution has been accumulated.
    pending = {}
    for node in trace:
        for a in node.args_:
            pending[id(a)] = pending.get(id(a), 0) + 1
    # (also left on the nodes for VJPs that fuse work across an edge only when it is the only one)
    for node in trace:
        node._consumers = pending.get(id(node), 0)
    prev, prev_wanted = _state.create_graph, _state.grad_wanted
    _state.create_graph = bool(create_graph)
    _state.grad_wanted = wanted      # (the VJPs with expensive operands consult state.wants_grad)
    try:
        for curr in reversed(trace):
            primals = curr.args_
            if not primals:
                continue
            if wanted is not None and id(curr) not in wanted:
                continue
            grads = curr.vjp_(primals, curr.grad(), curr)
            for primal, g in zip(primals, grads):
                if not primal.requires_grad() or (wanted is not None and id(primal) not in wanted):
                    continue
                if primal.has_grad():
                    g = add(g, primal.grad())
                primal.grad_(g)
                if not create_graph:
                    g.clear_args()
                hook = getattr(primal, "grad_hook", None)
                if hook is not None and not primal.args_ and pending[id(primal)] == 1:
                    hook(primal, g)      # a leaf's gradient is complete: e.g. start its all-reduce
                pending[id(primal)] -= 1
    finally:
        _state.create_graph = prev
        _state.grad_wanted = prev_wanted
        reset_node_id_recursive(out)


def jvp(out, inputs, tangents):
    """Forward mode: the tangent of `out` for the given tangents of `inputs`, by one walk over the
    graph in evaluation order that calls every node's `jvp` rule (the slot the reference's ops fill,
    e.g. tanh_op.mojo:56-73; the reference has no driver that calls them). Nodes that do not depend
    on `inputs` have a zero tangent."""
    from ..functional.init_ops import zeros_like
    tan = {id(x): t for x, t in zip(inputs, tangents)}
    for node in top_order(out):
        node.id = -1
        if id(node) in tan or not node.args_:
            continue
        ts = [tan.get(id(a)) for a in node.args_]
        if all(t is None for t in ts):
            continue
        if node.jvp_ is None:
            raise ValueError("jvp: op %r has no forward-mode rule" % (node.name,))
        ts = [t if t is not None else zeros_like(a) for t, a in zip(ts, node.args_)]
        tan[id(node)] = node.jvp_(node.args_, ts)
    res = tan.get(id(out))
    return res if res is not None else zeros_like(out)


def grad(outs=None, inputs=None, retain_grads=True, create_graph=False, argnums=(-1,)):
    """Two forms, as in the reference:
      grad(outs=[...], inputs=[...], retain_grads, create_graph) -> list of gradient Arrays
        (imperative, autograd/functional.mojo:70-97: stale gradients are cleared first);
      grad(f, argnums) -> Callable computing the gradient of f (:100-127)."""
    if callable(outs) or isinstance(outs, Callable):
        return _grad_transform(outs, list(argnums) if inputs is None else list(inputs))
    for out in outs:
        remove_grad_rec(out)
    for inp in inputs:
        remove_grad_rec(inp)
    for out in outs:
        jacrev(out, create_graph, only_for=inputs)
    final = []
    for inp in inputs:
        g = inp.grad()
        if not create_graph:
            g.clear_args()
            g.remove_grad()
        if not retain_grads:
            inp.remove_grad()
        final.append(g)
    return final


class Callable:
    """Functional-transform driver, eager branch (compile/callable.mojo:60-197)."""

    def __init__(self, func, argnums, order_of_differentiation=1, optimize_jit=False,
                 keep_intermediate_outs=False):
        self.func = func
        self.argnums = [list(a) for a in argnums]
        self.order_of_differentiation = order_of_differentiation
        self.keep_intermediate_outs = keep_intermediate_outs

    def __call__(self, args):
        from ..functional._utils import copy
        single = not isinstance(args, (list, tuple))
        arg_list = [args] if single else list(args)
        adapted = []
        for i, a in enumerate(arg_list):
            arg = a if len(a.args_) == 0 else copy(a)
            for order in range(self.order_of_differentiation):
                if i in self.argnums[order] or self.argnums[order][0] == -1:
                    arg.requires_grad_(True)
            adapted.append(arg)
        res = self.func(adapted[0]) if single else self.func(adapted)
        outs = [res]
        next_outs = [res]
        counts = [1]
        for order in range(self.order_of_differentiation):
            tmp, next_outs = next_outs, []
            for arr in tmp:
                arr.backward(create_graph=order < self.order_of_differentiation - 1)
                for i, a in enumerate(adapted):
                    if i in self.argnums[order] or self.argnums[order][0] == -1:
                        next_outs.append(a.grad())
                remove_grad_rec(arr)
            if self.keep_intermediate_outs:
                outs.extend(next_outs)
                counts.append(len(next_outs))
            else:
                outs = next_outs
        final = [copy(o) for o in outs]
        if len(final) == 1:
            return final[0]
        if self.keep_intermediate_outs:
            grouped, idx = [], 0
            for c in counts:
                grouped.append(final[idx:idx + c])
                idx += c
            return grouped
        return final


def _grad_transform(f, argnums):
    if isinstance(f, Callable):
        return Callable(f.func, f.argnums + [list(argnums)], f.order_of_differentiation + 1, False, False)
    return Callable(f, [list(argnums)], 1, False, False)


def jacobian(f, argnums=(-1,)):
    """jacobian(f)(x): same driver as grad; non-scalar outputs are seeded with an identity so the
    result is the full Jacobian (autograd/functional.mojo:130-149). Passing Arrays as the second
    argument evaluates immediately (:196-218)."""
    if _is_arrays(argnums):
        return _grad_transform(f, [-1])(argnums)
    return _grad_transform(f, list(argnums))


def hessian(f, argnums=(-1,)):
    if _is_arrays(argnums):
        return hessian(f)(argnums)
    return _grad_transform(_grad_transform(f, list(argnums)), list(argnums))


def value_and_grad(f, argnums=(-1,)):
    if isinstance(f, Callable):
        return Callable(f.func, f.argnums + [list(argnums)], f.order_of_differentiation + 1, False, True)
    return Callable(f, [list(argnums)], 1, False, True)


def _is_arrays(x):
    from .._array import Array
    return isinstance(x, Array) or (isinstance(x, (list, tuple)) and x and isinstance(x[0], Array))
