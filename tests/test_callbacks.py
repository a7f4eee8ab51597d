# SPDX-License-Identifier: Apache-2.0
import pytest

from arctictraining_b200.callback.mixin import CallbackMixin
from arctictraining_b200.callback.mixin import callback_wrapper


def test_pre_callback_rewrites_args_and_post_rewrites_return():
    def double_x(self, x):
        return x * 2

    def plus_one(self, result):
        return result + 1

    class Thing(CallbackMixin):
        callbacks = [("pre-compute", double_x), ("post-compute", plus_one)]

        @callback_wrapper("compute")
        def compute(self, x: int, y: int = 1) -> int:
            return x + y

    assert Thing().compute(3) == 3 * 2 + 1 + 1
    assert Thing().compute(3, y=10) == 6 + 10 + 1


def test_pre_callback_with_two_args_must_return_both_in_order():
    def swap(self, a, b):
        return b, a

    def wrong(self, a, b):
        return a

    class Ok(CallbackMixin):
        callbacks = [("pre-f", swap)]

        @callback_wrapper("f")
        def f(self, a, b) -> str:
            return f"{a}{b}"

    assert Ok().f("x", "y") == "yx"

    class Bad(CallbackMixin):
        callbacks = [("pre-f", wrong)]

        @callback_wrapper("f")
        def f(self, a, b) -> str:
            return f"{a}{b}"

    with pytest.raises((ValueError, TypeError)):
        Bad().f("x", "y")


def test_method_named_callbacks_and_none_returning_methods():
    calls = []

    class Thing(CallbackMixin):
        @callback_wrapper("act")
        def act(self) -> None:
            calls.append("act")

        def pre_act_callback(self):
            calls.append("pre")

        def post_act_callback(self):
            calls.append("post")

    Thing().act()
    assert calls == ["pre", "act", "post"]


def test_overridden_method_is_rewrapped_and_callbacks_accumulate_across_two_levels():
    log = []

    def base_cb(self, v):
        log.append("base")
        return v

    def child_cb(self, v):
        log.append("child")
        return v

    class Base(CallbackMixin):
        callbacks = [("post-go", base_cb)]

        @callback_wrapper("go")
        def go(self, n: int) -> int:
            return n

    class Child(Base):
        callbacks = [("post-go", child_cb)]

        def go(self, n: int) -> int:  # override without decorating again
            return n * 10

    class GrandChild(Child):
        def go(self, n: int) -> int:
            return n * 100

    assert Child().go(1) == 10
    assert log == ["base", "child"]
    log.clear()
    assert GrandChild().go(1) == 100
    assert log == ["base", "child"]


def test_invalid_callbacks_are_rejected():
    def with_default(self, x=1):
        return x

    def unknown_param(self, nope):
        return nope

    class A(CallbackMixin):
        callbacks = [("pre-m", with_default)]

        @callback_wrapper("m")
        def m(self, x) -> int:
            return x

    class B(CallbackMixin):
        callbacks = [("pre-m", unknown_param)]

        @callback_wrapper("m")
        def m(self, x) -> int:
            return x

    class C(CallbackMixin):
        callbacks = [("pre-missing", lambda self: None)]

        @callback_wrapper("m")
        def m(self, x) -> int:
            return x

    for cls in (A, B, C):
        with pytest.raises(ValueError):
            cls()


def test_init_is_an_event():
    seen = []

    class Thing(CallbackMixin):
        def __init__(self, v):
            self.v = v

        def post_init_callback(self):
            seen.append(self.v)

    Thing(5)
    assert seen == [5]


def test_callbacks_run_once_when_an_override_calls_super():
    from arctictraining_b200.callback.mixin import CallbackMixin
    from arctictraining_b200.callback.mixin import callback_wrapper

    seen = []

    class Base(CallbackMixin):
        @callback_wrapper("make")
        def make(self, x):
            return x + 1

        def post_make_callback(self, result):
            seen.append(result)
            return result * 10

    class Child(Base):
        def make(self, x):
            return super().make(x) + 100  # the parent's wrapper must not run the callbacks a second time

    assert Child().make(1) == 1020 and seen == [102]
    assert Base().make(1) == 20
    obj = Child()
    assert obj.make(2) == 1030 and obj.make(2) == 1030  # the running-set is cleared after each call
