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
