"""Block input/output contracts (mirrors src/cache_dit/caching/forward_pattern.py:4-93).

A pattern says what a transformer block takes and returns:
  Pattern_0: (hidden, encoder) -> (hidden, encoder)      Pattern_3: (hidden) -> hidden
  Pattern_1: (hidden, encoder) -> (encoder, hidden)      Pattern_4: (hidden) -> (hidden, encoder)
  Pattern_2: (hidden, encoder) -> hidden                 Pattern_5: (hidden) -> (encoder, hidden)
"""
from enum import Enum

_HE = ("hidden_states", "encoder_hidden_states")
_EH = ("encoder_hidden_states", "hidden_states")
_H = ("hidden_states", )


class ForwardPattern(Enum):

  def __init__(self, Return_H_First, Return_H_Only, Forward_H_only, In, Out, Supported):
    self.Return_H_First = Return_H_First
    self.Return_H_Only = Return_H_Only
    self.Forward_H_only = Forward_H_only
    self.In = In
    self.Out = Out
    self.Supported = Supported

  Pattern_0 = (True, False, False, _HE, _HE, True)
  Pattern_1 = (False, False, False, _HE, _EH, True)
  Pattern_2 = (False, True, False, _HE, _H, True)
  Pattern_3 = (False, True, True, _H, _H, True)
  Pattern_4 = (True, False, True, _H, _HE, True)
  Pattern_5 = (False, False, True, _H, _EH, True)

  @staticmethod
  def supported_patterns():
    return [p for p in ForwardPattern if p.Supported]
