"""Stop strings: end a completion when its detokenised text contains one of the given strings.

The engine works on token ids, so the match runs where the text is made (the offline ``LLM`` loop and the
server's stream).  A stop string can straddle token boundaries, and a stream must not send text that later
turns out to be the beginning of a stop string: the matcher holds back the last ``longest stop - 1``
characters until more text arrives or the request ends.
"""
from __future__ import annotations


class StopStringMatcher:
    def __init__(self, stops, include_in_output: bool = False):
        self.stops = [s for s in (stops or []) if s]
        self.include = include_in_output
        self.hold = max((len(s) for s in self.stops), default=1) - 1
        self.sent = 0                # characters handed out so far
        self.hit = None              # the stop string that ended the text

    def push(self, text: str, final: bool = False):
        """``text`` is the whole completion so far.  Returns (new text that may be shown, stopped)."""
        if self.hit is not None:
            return "", True
        best = None
        for s in self.stops:
            i = text.find(s, max(0, self.sent - len(s) + 1))
            if i >= 0 and (best is None or i < best[0]):
                best = (i, s)
        if best is not None:
            end = best[0] + (len(best[1]) if self.include else 0)
            delta, self.sent, self.hit = text[self.sent:max(end, self.sent)], max(end, self.sent), best[1]
            return delta, True
        safe = len(text) if final else max(self.sent, len(text) - self.hold)
        delta, self.sent = text[self.sent:safe], safe
        return delta, False


def truncate_at_stop(text: str, stops, include_in_output: bool = False):
    """(text cut at the first stop string, the stop string or None)."""
    m = StopStringMatcher(stops, include_in_output)
    out, _ = m.push(text, final=True)
    return out, m.hit
