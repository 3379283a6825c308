"""Decision models: one forward pass answers typed questions about a state.

A request is a state (token ids) and named questions - a ``Choice`` among named options or a ``Score`` on a numeric scale
(scored as a choice over its buckets).  The questions are laid out behind the state in one row (``layout_row``), a backbone
reads the row, a ``DecisionHead`` scores every option of every question at that question's marker position, and the answer
is a distribution over exactly the options the question names.  ``DecisionObjective`` trains with proper scoring rules
(log score or Brier); ``Temperatures`` / ``binning`` / ``Abstention`` calibrate and gate the answers.

Reference: src/dew/decision/{questions,layout,head,objective,calibration,task}.py (23 files, 12.1 K lines).
"""
from .questions import Choice, Question, Score
from .model import DecisionHead, Decide, layout_row
from .objective import DecisionObjective
from .calibration import Abstention, Temperatures, binning

__all__ = ["Abstention", "Choice", "Decide", "DecisionHead", "DecisionObjective", "Question", "Score", "Temperatures", "binning", "layout_row"]
