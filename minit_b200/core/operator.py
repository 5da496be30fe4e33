"""Operator records (reference: minit/core/operator.py:4-6)."""


class Operator:
    def type(self):
        return type(self)
