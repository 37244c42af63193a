from __future__ import annotations

import pytest

from tpu_cake_b200.run_ledger import RunLedger, RunState

RUN = "a" * 64


def test_legal_path_and_idempotent_completion(tmp_path):
    with RunLedger(tmp_path / "ledger.sqlite", clock_ns=iter(range(1, 100)).__next__) as ledger:
        ledger.create(RUN, {"m": 128})
        for state in (RunState.VERIFIED, RunState.LOWERED, RunState.COMPILED, RunState.CORRECT, RunState.TIMED):
            ledger.transition(RUN, state, {"state": state.value})
        again = ledger.transition(RUN, RunState.TIMED, {"state": "timed"})
        assert again.sequence == 6 and ledger.current_state(RUN) is RunState.TIMED
        with pytest.raises(ValueError, match="conflicting duplicate"):
            ledger.transition(RUN, RunState.TIMED, {"state": "different"})
        assert [e.state for e in ledger.history(RUN)][0] is RunState.CREATED


def test_illegal_transitions_and_terminal_states(tmp_path):
    with RunLedger(tmp_path / "ledger.sqlite") as ledger:
        with pytest.raises(ValueError, match="does not exist"):
            ledger.transition(RUN, RunState.VERIFIED, {})
        ledger.create(RUN, {})
        with pytest.raises(ValueError, match="invalid run transition created -> compiled"):
            ledger.transition(RUN, RunState.COMPILED, {})
        ledger.transition(RUN, RunState.REJECTED, {"reason": "numerical mismatch"})
        with pytest.raises(ValueError, match="already terminal"):
            ledger.transition(RUN, RunState.VERIFIED, {})
