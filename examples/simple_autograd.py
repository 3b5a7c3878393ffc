"""Gradients of small expressions (ferrum-examples/src/simple_autograd.rs): z = sum(x * y + x^2)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403,E402


def main():
    x = Tensor.from_slice([1.0, 2.0, 3.0]).set_requires_grad(True)
    y = Tensor.from_slice([4.0, 5.0, 6.0]).set_requires_grad(True)
    z = x.mul(y).add(x.pow(2.0)).sum()
    z.backward()
    print("z      =", z.item())
    print("dz/dx  =", x.grad().to_vec(), "(expected y + 2x = [6, 9, 12])")
    print("dz/dy  =", y.grad().to_vec(), "(expected x = [1, 2, 3])")
    with no_grad():
        w = x.mul(y)
    print("inside no_grad: requires_grad =", w.requires_grad())
    ok = fb.autograd.quick_gradcheck(lambda t: t.tanh().mul(t).sum(), Tensor.randn([5]))
    print("gradcheck tanh(t) * t:", ok)
    return x.grad().to_vec(), y.grad().to_vec()


if __name__ == "__main__":
    main()
