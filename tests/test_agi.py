import math
import threading

import pytest
import torch

from transformers_fusion_b200 import agi
from transformers_fusion_b200.agi.core import KnowledgeDistillation
from transformers_fusion_b200.utils.inferno import InfernoCounter, TaskQueue, inferno_metric


def echo(prompt):
    if "Critique" in prompt:
        return "approve: no issues"
    if "numbered steps" in prompt:
        return "1. gather data\n2. train model (after 1)\n3. evaluate (after 2)\n4. write report (after 2, 3)"
    return "result for " + prompt[:30]


def test_monitor_reflector_metacognition():
    mon = agi.SelfMonitor(logits=lambda p: torch.tensor([5.0, 0.0, 0.0, 0.0]))
    st = mon.analyze("q", "a")
    assert st.confidence > 0.9 and 0 <= st.uncertainty < 0.2
    flat, peaked = torch.zeros(1, 8), torch.tensor([[9.0] + [0.0] * 7])
    assert mon.distribution_shift(flat, flat) < 1e-9 and mon.detect_drift(peaked, flat) and mon.get_recent_alerts()[0].source == "drift"
    r = agi.SelfReflector(echo)
    assert r.refine("x", "No issues found") == "x" and r.consistency_check("a b c", "a b d") == 0.5
    assert r.ece_calibration([0.9, 0.9, 0.1, 0.1], [True, True, False, False]) == pytest.approx(0.1)
    assert r.identify_errors("p", "", "x y") == ["empty output", "missing: x y"]
    mc = agi.MetaCognition()
    ens = torch.stack([torch.tensor([4.0, 0, 0]), torch.tensor([0, 4.0, 0])])
    assert mc.epistemic_uncertainty(ens) > 0.3 and mc.epistemic_uncertainty(ens[0]) < 1e-6
    assert mc.reasoning_quality(["add the numbers", "the numbers sum to five"]) > 0.7 and mc.reasoning_quality([]) == 0
    mc.self_model_update("q", 0.9, True)
    mc.self_model_update("q", 0.9, False)
    assert mc.self_model_accuracy == 0.5


def test_guardrails_sandbox_verifier():
    g = agi.SafetyGuardrails()
    assert g.check_input("please summarise this") and not g.check_output("run rm -rf / now")
    assert not g.check_modification("guardrail rules", "relax") and g.check_modification("learning rate", "halve it")
    g.set_invariant("positive", lambda: 3 > 2)
    assert g.check_invariant("positive") and not g.check_invariant("missing")
    g.set_kill_switch(True)
    assert not g.check_input("anything") and g.is_killed() and len(g.get_audit_log()) >= 6
    sb = agi.Sandbox()
    assert sb.static_analysis("import os\nopen('x')") == ["import of 'os' is not allowed", "call to 'open' is not allowed"]
    assert "syntax error" in sb.static_analysis("def (")[0] and sb.static_analysis("while True:\n    pass") == ["unbounded 'while True' loop"]
    r = sb.compile_and_test("def sq(x):\n    return x * x\n", ["sq(3) == 9", "sq(-2) == 4", "sq(2) == 5"])
    assert r.compiled and r.tests_passed == 2 and r.tests_total == 3
    assert not sb.compile_and_test("import socket", ["True"]).compiled
    slow = sb._run("x = 0\nwhile x < 10**12:\n    x += 1\n", 0.5)
    assert slow.timed_out or slow.exit_code != 0                       # bounded: never runs away
    v = agi.SelfVerifier(sb)
    assert v.verify_arithmetic("2 * (3 + 4)", 14) and not v.verify_arithmetic("__import__('os')", 0)
    assert v.verify_code("def f(x):\n    return x + 1\n", ["f(1) == 2"])


def test_agents_planning_flywheel():
    co = agi.MultiAgentCoordinator(echo)
    out = co.run_task("sort a list")
    assert out.startswith("result for [Synthesizer]") and co.is_converged() and co.get_round() == 1
    assert co.get_message_queue(co.IMPLEMENTER)[0].sender == co.ANALYST and len(co.get_agent_history(co.CRITIC)) == 1
    pe = agi.PlanningEngine(echo)
    plan = pe.plan("ship a model")
    assert [s.id for s in plan] == [1, 2, 3, 4] and plan[3].depends_on == [2, 3] and pe.execute(plan) and len(pe.execution_history) == 4
    with pytest.raises(ValueError):
        pe.topological_sort([agi.PlanStep(1, "a", [2]), agi.PlanStep(2, "b", [1])])
    fail = agi.PlanningEngine(None, executor=lambda s: s.id != 2)
    p2 = fail.plan("a then b then c")
    assert not fail.execute(p2)
    rp = fail.replan(p2, "b failed")
    assert rp[0].done and rp[1].description == "resolve: b failed" and rp[2].depends_on == [rp[1].id]
    # flywheel: the "model" improves when the improver teaches it the failing cases
    known = {}
    h = agi.EvaluationHarness(lambda p: known.get(p, "?"))
    fw = agi.Flywheel(h, lambda fails: known.update({p: e for p, _, e in fails}))
    its = fw.run([("2+2", "4"), ("capital of France", "Paris")], max_iterations=3)
    assert [i["accuracy"] for i in its] == [0.0, 1.0]
    hitl = agi.HITL(lambda a: False)
    assert len(agi.Flywheel(agi.EvaluationHarness(lambda p: "?"), lambda f: None, hitl=hitl).run([("a", "b")], 3)) == 1
    imp = agi.RecursiveSelfImprover(lambda s: -abs(math.log10(s["learning_rate"]) + 3))     # best at 1e-3
    imp.improvement_cycle(8)
    assert 4e-4 < imp.settings["learning_rate"] < 2e-3


def test_misc_components():
    ex = agi.CuriosityDrivenExplorer()
    for _ in range(10):
        ex.observe("known", 1.0, 1.0)
    ex.observe("surprising", 0.0, 5.0)
    assert ex.select(["known", "surprising"]) == "surprising" and ex.select(["known", "new"]) == "new"
    kd = KnowledgeDistillation(2.0, 0.5)
    t = torch.randn(4, 10)
    assert float(kd.loss(t, t)) < 1e-6 and float(kd.loss(torch.randn(4, 10), t, torch.randint(0, 10, (4,)))) > 0
    tools = agi.ToolUse()
    tools.register("double", lambda a: int(a) * 2)
    assert tools.run("first double(21) then unknown(3) then double(x)") == {"double(21)": 42, "double(x)": "error: invalid literal for int() with base 10: 'x'"}
    mem = agi.MemorySystem(2)
    for s in ("the cat sat", "dogs bark loudly", "cats purr softly", "rain falls"):
        mem.remember(s)
    assert mem.recall("cat sat on", 1) == ["the cat sat"] and len(mem.long) == 2
    chain, ans = agi.ChainOfThought(lambda p: "therefore 4" if "Step 2" in p else "add").solve("2+2", 5)
    assert chain == ["add", "therefore 4"]
    best, _ = agi.PromptOptimizer(lambda s: len(s)).optimize("task", ["{base}!", "Please do: {base} carefully"])
    assert best.startswith("Please")
    assert 0 <= agi.AlignmentSystem().value_alignment_score("I will help and explain safely") <= 1
    assert agi.AlignmentSystem().value_alignment_score("exploit and steal") < agi.AlignmentSystem().value_alignment_score("help explain")


def test_meta_engine_multi_agent_system_eval_world():
    me = agi.MetaCognitionEngine(5)
    for c, ok in [(0.9, True)] * 8 + [(0.9, False)] * 2 + [(0.3, False)] * 5:
        me.record_confidence(c, ok)
    assert me.expected_calibration_error() == pytest.approx((10 * 0.1 + 5 * 0.3) / 15) and me.calibrate(0.9) == pytest.approx(0.8)
    gid, kids = me.decompose_goal("ship", ["build", "test"])
    me.complete(kids[0])
    assert me.progress(gid) == 0.5
    me.complete(kids[1])
    assert me.goals[gid].done and me.assess().goals_completed == 1.0
    ch = me.begin_chain("g")
    me.add_step(ch, "a", 0.9), me.add_step(ch, "b", 0.5)
    assert ch.confidence() == pytest.approx(0.45) and me.weakest_step(ch).content == "b"
    mas = agi.MultiAgentSystem()
    a = mas.add_agent("worker", lambda p: "done:" + p[:12], 1.0)
    b = mas.add_agent("worker", lambda p: "blue", 3.0)
    t0 = mas.add_subtask("collect")
    t1 = mas.add_subtask("analyse", [t0])
    assert mas.run() and mas.subtasks[t1].done and mas.read(f"subtask/{t0}") is not None
    win, tally, votes = mas.vote("colour?", ["red", "blue"])
    assert win == "blue" and tally["blue"] == 3.0
    mas.broadcast(a, "note", "hello")
    assert mas.receive(b, "note").content == "hello" and mas.receive(b) is None
    assert agi.pass_at_k(5, 0, 1) == 0 and agi.pass_at_k(5, 5, 1) == 1 and agi.pass_at_k(10, 3, 2) == pytest.approx(1 - (7 * 6) / (10 * 9))
    suite = agi.SelfEvalSuite(lambda p: "4" if "2+2" in p.replace(" ", "").lower() else "?", lambda p, o: 0.9 if o == "4" else 0.1)
    rep = suite.evaluate([("what is 2+2", "4"), ("capital of France", "Paris")])
    assert rep.accuracy == 0.5 and rep.consistency == 1.0 and rep.ece == pytest.approx(0.1) and rep.pass_at_k[1] == 0.5
    better = agi.self_eval.EvaluationReport(accuracy=0.9, consistency=1.0, robustness=1.0, tokens_per_sec=rep.tokens_per_sec)
    assert agi.SelfEvalSuite.compare_versions(rep, better)["improved"]
    wm = agi.WorldModel()
    for _ in range(5):
        wm.observe("start", "right", "mid", 0.0)
        wm.observe("mid", "right", "goal", 10.0)
        wm.observe("start", "left", "pit", -5.0)
    assert wm.predict("start", "right").next_state == "mid" and wm.mpc_action("start", 3) == "right"
    plan = wm.plan_beam("start", 2)
    assert plan.actions == ["right", "right"] and plan.states == ["start", "mid", "goal"] and plan.expected_return == pytest.approx(9.5)
    cf = wm.counterfactual("start", ["left"], ["right", "right"])
    assert cf.difference == pytest.approx(14.5) and wm.uncertainty("start", "right")[0] < wm.uncertainty("nowhere", "right")[0]


def test_inferno():
    assert inferno_metric(1e21, 32) == pytest.approx(0.5) and inferno_metric(1e21, 4) == pytest.approx(4.0)
    c = InfernoCounter(8.0)
    c.start(), c.add_gemm(64, 64, 64), c.stop()
    assert c.ops == 2 * 64 ** 3 and c.flops() > 0 and c.inferno() == pytest.approx(inferno_metric(c.flops(), 8.0))
    gate = threading.Event()
    q = TaskQueue(workers=1)
    first = q.submit(gate.wait, priority=100)
    lo, hi = q.submit(lambda: "lo", priority=1), q.submit(lambda: "hi", priority=9)
    gate.set()
    assert hi.result(5) == "hi" and lo.result(5) == "lo" and q.order == [100, 9, 1]
    bad = q.submit(lambda: 1 / 0)
    with pytest.raises(ZeroDivisionError):
        bad.result(5)
    q.stop()


def test_world_model_reference_verbs():
    from transformers_fusion_b200.agi.world_model import Transition, WorldModel
    wm = WorldModel(discount=0.9)
    wm.train_on_transitions([Transition("a", "go", "b", 1.0), Transition("b", "go", "c", 5.0), Transition("a", "stay", "a", 0.1),
                             Transition("b", "stay", "b", 0.0), Transition("a", "go", "b", 1.0)])
    assert wm.simulate_step("a", "go") == "b" and wm.predict_reward("a", "go") == 1.0 and len(wm.get_transition_buffer()) == 5
    traj = wm.simulate_trajectory("a", ["go", "go", "go"])
    assert [t.next_state for t in traj] == ["b", "c"] and traj[1].reward == 5.0
    plan = wm.beam_search_plan("a", 2, beam_width=4)
    assert plan.actions == ["go", "go"] and abs(plan.expected_return - (1.0 + 0.9 * 5.0)) < 1e-9 and wm.plan_actions("a", 2) == ["go", "go"]
    mpc = wm.model_predictive_control("a", 2, n_samples=40)
    assert mpc.actions == ["go", "go"]
    wm.set_current_state("a")
    assert wm.get_current_state() == "a" and wm.plan(2) == ["a", "b", "c"]
    pr, unc = wm.predict_with_uncertainty("a", "go")
    assert pr.next_state == "b" and unc.epistemic_uncertainty < wm.estimate_uncertainty("zz", "go").epistemic_uncertainty
    assert unc.ensemble_size == 5 and unc.disagreement_magnitude == 0.0
    assert wm.compute_ensemble_disagreement(["x", "x", "y", "z"]) == 0.5 and wm.compute_ensemble_disagreement([]) == 0.0
    cf = wm.counterfactual_analysis("a", "stay", "go")
    assert cf.difference == pytest.approx(0.9) and len(wm.batch_counterfactual("a", "stay", ["go", "stay"])) == 2
    wm.store_state({"room": 1}, importance=0.2, key="room/kitchen", vector=[1.0, 0.0])
    wm.store_state({"room": 2}, importance=0.9, key="room/garden", vector=[0.0, 1.0])
    wm.store_state({"room": 3}, importance=0.1, key="hall", vector=[0.7, 0.7])
    assert wm.retrieve_most_relevant("room/gar")["room"] == 2 and wm.retrieve_most_relevant([0.9, 0.1])["room"] == 1
    wm.consolidate_memory(2)
    assert len(wm.get_memory()) == 2 and all(e["state"]["room"] != 3 for e in wm.get_memory())
    st = wm.get_stats()
    assert st["total_transitions"] == 5 and st["planning_calls"] >= 3 and st["memory_entries"] == 2 and st["total_predictions"] >= 2
    wm.reset_stats()
    assert wm.get_stats()["planning_calls"] == 0


def test_multi_agent_reference_verbs():
    from transformers_fusion_b200.agi.multi_agent import AgentMessage, MultiAgentSystem
    mas = MultiAgentSystem()
    flaky_calls = []

    def flaky(task):
        flaky_calls.append(task)
        raise RuntimeError("tool down")
    a0 = mas.add_agent("supervisor", lambda t: f"ok:{t}")
    a1 = mas.add_agent("worker", flaky)
    a2 = mas.add_agent("worker", lambda t: f"done:{t}")
    mas.configure("STAR")
    assert mas.agent_count() == 3 and mas.get_agent(a1).role == "worker"
    assert mas.communicate_direct(a0, a2, "hello") and not mas.communicate_direct(a1, a2, "side channel")      # spokes only reach the hub
    mas.set_max_queue_size(2)
    for i in range(4):
        mas.send_message(AgentMessage(a0, a2, "t", f"m{i}"))
    got = mas.receive_messages(a2)
    assert [m.content for m in got] == ["m2", "m3"] and mas.receive_messages(a2) == [] and len(mas.get_histories()) == 5
    mas.configure("RING")
    assert mas.communicate_direct(a1, a2, "neighbour")
    plan = mas.create_plan("load the data; clean it, then train the model. evaluate", 4)
    assert plan.high_level_steps == ["load the data", "clean it", "train the model", "evaluate"] and len(mas.get_ready_subtasks()) == 1
    assert mas.get_task_status(plan.subtask_ids[0]) == "pending" and mas.get_task_status(99) == "unknown"
    mas.assign_subtask(plan.subtask_ids[0], a1)                        # the flaky agent gets the first step
    assert mas.get_task_status(plan.subtask_ids[0]) == "assigned"
    assert mas.execute_plan(plan, max_rounds=12) and plan.completed and mas.get_plan_progress(plan) == 1.0
    assert flaky_calls and mas.get_metrics(a1).tasks_failed >= 1 and mas.subtasks[plan.subtask_ids[0]].result.startswith(("ok:", "done:"))
    assert len(mas.search_blackboard("subtask/")) == 4 and mas.read_blackboard("subtask/0") != "" and mas.read_blackboard("nope") == ""
    mas.write_blackboard("note", "v1", a0), mas.write_blackboard("note", "v2", a2)
    assert mas.supervisor_resolve_conflicts() == ["note"]
    mas.cleanup_blackboard()
    assert all(k.startswith("plan/") for k in mas.blackboard)
    mas.submit_vote(a0, "ship", True, 0.9, "tests pass"), mas.submit_vote(a1, "ship", False, 0.2), mas.submit_vote(a2, "ship", True, 0.8)
    assert mas.check_consensus(0.6) and len(mas.get_votes()) == 3
    mas.reset_votes()
    assert not mas.check_consensus()
    t = mas.assign_task_to_role("worker", "extra job")
    assert mas.subtasks[t].assigned_to in (a1, a2) and mas.run_episode(3) >= 1 and mas.get_task_status(t) == "done"
    mas.update_metrics(a2)
    assert not mas.get_agent(a2).busy and "agent 2 (worker)" in mas.metrics_summary() and len(mas.get_all_metrics()) == 3
    mas.supervisor_escalate("budget exceeded")
    assert mas.escalations == ["budget exceeded"] and mas.search_blackboard("escalation/")
    t2 = mas.assign_task(a2, "last job")
    mas.remove_agent(a2)
    assert mas.agent_count() == 2 and mas.subtasks[t2].assigned_to == -1 and mas.run_round(3)


def test_self_eval_suite_reference_verbs():
    import re
    from transformers_fusion_b200.agi.self_eval import SelfEvalSuite

    def solver(prompt):                                   # answers the generated benchmarks exactly
        nums = list(map(int, re.findall(r"\d+", prompt.split("(A)")[0] if "(A)" in prompt else prompt)))
        if "(A)" not in prompt:
            return str(sum(nums[:2])) if len(nums) >= 2 else "0"
        a, b = nums[:2]
        right = a * b if "times" in prompt.lower() else (a + b if "plus" in prompt.lower() else max(a, b))
        opts = dict(re.findall(r"\((\w)\) (\d+)", prompt))
        return next((f"({l})" for l, v in opts.items() if int(v) == right), "(A)")
    s = SelfEvalSuite(solver, confidence=lambda p, o: 0.95)
    for fn in (s.run_accuracy_benchmark_mmlu, s.run_accuracy_benchmark_arc, s.run_accuracy_benchmark_gsm8k):
        r = fn(12)
        assert r["n_total"] == 12 and r["accuracy"] >= 0.9, r
    cal = s.run_calibration_benchmark(20)
    assert cal["bins"][9]["count"] == 20 and cal["ece"] == pytest.approx(abs(cal["bins"][9]["accuracy"] - 0.95))
    assert SelfEvalSuite.compute_expected_calibration_error([{"count": 10, "accuracy": 0.5, "confidence": 0.9}, {"count": 0, "accuracy": 0, "confidence": 0}]) == pytest.approx(0.4)
    c = s.run_consistency_benchmark("Ann has 3 apples and buys 4 more.", 4)
    assert c["agreement"] == 1.0 and c["majority_answer"] == "7" and len(s.run_consistency_suite(3, 2)) == 3
    rb = s.run_robustness_suite(3, 4)
    assert len(rb) == 3 and all(0.0 <= r["stability"] <= 1.0 for r in rb)
    assert s.run_speed_benchmark(5)["ops_per_sec"] > 0 and s.run_memory_benchmark(2)["peak_bytes"] > 0
    assert s.run_pass_at_k("gsm8k", 2, 4)["pass_at_k"] == 1.0 and [r["k"] for r in s.run_pass_at_k_suite(5, n_problems=2)] == [1, 2, 5]
    s.register_benchmark("mine", [("What is 1 plus 1? (A) 2 (B) 3", "(A)")])
    assert s.run_accuracy_benchmark("mine", 5)["n_total"] == 1
    rep = s.generate_report("v1", n_samples=6)
    assert rep["version_id"] == "v1" and 0.8 < rep["overall_score"] <= 1.0 and s.get_latest_report() is rep and len(s.get_report_history()) == 1
    weak = SelfEvalSuite(lambda p: "no idea")
    assert weak.run_accuracy_benchmark_gsm8k(5)["accuracy"] == 0.0


def test_meta_cognition_reference_verbs():
    from transformers_fusion_b200.agi.meta import FeedbackEntry, MetaCognitionEngine
    m = MetaCognitionEngine()
    chain = m.analyze_reasoning("What is the value of x?", "We set x = 3. Maybe the value matters. Then x = 4. So the answer is four.")
    assert len(chain.steps) == 4 and chain.steps[1].confidence < chain.steps[0].confidence        # hedged step
    assert m.find_first_error_step(chain) == 2 and "contradicts step 0" in m.diagnose_error(chain, 2)
    assert m.calculate_chain_consistency(chain) < 1.0 and m.diagnose_error(chain, 9) == "no error step"
    from transformers_fusion_b200.agi.meta import ReasoningStep
    assert not m.check_step_consistency(ReasoningStep(0, "the sky is blue"), ReasoningStep(1, "the sky is not blue"))
    assert m.check_step_consistency(ReasoningStep(0, "the sky is blue"), ReasoningStep(1, "grass is green"))
    for i in range(20):
        m.record_confidence(0.9, i % 2 == 0, "math")
    assert m.get_expected_calibration_error() == pytest.approx(0.4) and len(m.get_calibration_bins(5)) == 5
    assert m.get_current_confidence() == pytest.approx(0.5) and len(m.get_confidence_history()) == 20      # calibrated down from 0.9
    d = m.decompose("collect the logs; parse them, then write the report", 5)
    assert len(d.subgoals) == 3 and m.get_ready_subgoals(d) == [d.subgoals[0]] and not m.check_subgoal_completion(d)
    m.complete(d.subgoals[0])
    assert m.get_ready_subgoals(d) == [d.subgoals[1]]
    for g in d.subgoals[1:]:
        m.complete(g)
    assert m.check_subgoal_completion(d) and m.goals[d.root].done
    assert m.select_strategy("solve 12 * 7", 0.3) == "CHAIN_OF_THOUGHT" and m.select_strategy("solve 12 * 7", 0.6) == "VERIFY_THEN_ANSWER"
    assert m.select_strategy("say hello", 0.1) == "DIRECT" and m.select_strategy("anything", 0.9) == "DECOMPOSE"
    for ok in (False, False, True):
        m.record_feedback(FeedbackEntry("calculate 3 + 4", "DIRECT", 1.0 if ok else 0.0, ok, "" if ok else "arithmetic slip"))
    m.record_feedback(FeedbackEntry("solve 9 - 2", "VERIFY_THEN_ANSWER", 0.9, True))
    assert m.get_best_strategy_for_task_type("math") == "VERIFY_THEN_ANSWER" and m.select_strategy("solve 1 + 1", 0.1) == "VERIFY_THEN_ANSWER"
    pats = m.extract_improvement_patterns()
    assert "recurring failure: arithmetic slip (x2)" in pats and any("DIRECT fails" in p for p in pats)
    assert "4 tasks, 2 succeeded" in m.generate_feedback_summary() and len(m.get_recent_feedback(2)) == 2
    a = m.assess_self(10)
    assert a.overconfidence == pytest.approx(0.4) and any("recurring" in i for i in a.insights)
    ins = m.generate_insight("why is the sky blue", "Because of scattering. It is blue = 1. It is blue = 2.")
    assert ins["task_type"] == "explanation" and ins["first_error_step"] == 2 and ins["consistency"] < 1
    assert len(m.get_history()) >= 2
    m.reset()
    assert m.get_history() == [] and m.generate_feedback_summary() == "no feedback recorded"


def test_core_classes_reference_verbs():
    import torch
    from transformers_fusion_b200.agi import core as A
    rs = A.RollingStats()
    for v in (1.0, 1.1, 0.9, 1.0, 1.05, 0.95, 1.0, 1.0, 1.02):
        rs.update(v)
    assert rs.is_anomalous(5.0) and not rs.is_anomalous(1.01) and rs.z_score(1.0) == pytest.approx(rs.zscore(1.0))
    mon = A.SelfMonitor()
    assert mon.get_confidence_stats() is mon.confidence_stats and mon.get_uncertainty_stats() is mon.uncertainty_stats
    mc = A.MetaCognition()
    mc.self_model_update("q", 0.9, True), mc.self_model_update("q", 0.9, False)
    assert mc.get_self_model_accuracy() == 0.5
    g = A.SafetyGuardrails()
    g.set_paused(True)
    assert g.is_paused()
    h = A.HITL(lambda a: True)
    h.request_approval("deploy"), h.pause()
    assert h.is_paused() and not h.request_approval("again") and len(h.get_approval_history()) == 2
    pe = A.PlanningEngine()
    plan = pe.plan("read the file; parse it")
    pe.execute(plan)
    assert len(pe.get_execution_history()) == len(plan) >= 2
    # self-improver knobs: the evaluation prefers a learning rate near 2e-4 and some dropout
    score = lambda s: -abs(math.log(s["learning_rate"] / 2e-4)) - abs(s["dropout"] - 0.05)
    imp = A.RecursiveSelfImprover(score)
    assert imp.self_modify("training is slow and has reached a plateau") and imp.settings["learning_rate"] == pytest.approx(1.5e-4)
    assert imp.self_modify("add dropout") and imp.settings["dropout"] == 0.05
    assert not imp.self_modify("nothing to change here")
    kept = dict(imp.settings)
    assert not imp.self_modify("loss is unstable and diverging") and imp.settings == kept          # halving the rate scores worse: rolled back
    imp.apply_pruning(0.02), imp.apply_perturbation(0.03)
    assert imp.settings["prune_threshold"] == 0.02 and imp.settings["perturbation"] == 0.03
    assert imp.adjust_format("memory bandwidth bound") == "q4" and imp.adjust_format("accuracy degraded") == "q8"
    assert imp.evaluate_candidate({**imp.settings, "learning_rate": 2e-4}) > imp.evaluate_candidate(imp.settings)
    sv = A.SelfVerifier()
    assert sv.verify("what is 12 * 7", "12 * 7 = 84") and not sv.verify("what is 12 * 7", "12 * 7 = 85") and not sv.verify("x", "  ")
    assert sv.verify("write code", "```python\nprint(sum(range(4)))\n```") and not sv.verify("write code", "```python\nraise SystemExit(3)\n```")
    ec = sv.find_edge_cases("sort the list and divide by 10")
    assert {"division by zero", "already sorted", "9", "10", "11", "empty input"} <= set(ec)
    ex = A.CuriosityDrivenExplorer()
    visits = ex.explore(12, ["a", "b", "c"], outcome=lambda k: {"a": 0.0, "b": 0.0, "c": 5.0}[k])
    assert len(visits) == 12 and visits.count(2) > visits.count(0) and ex.intrinsic_reward("c") > ex.intrinsic_reward("a")
    assert ex.intrinsic_reward(torch.ones(3)) > 0
    learn_log = []
    cl = A.ContinuousLearner(lambda b: learn_log.append(b) or 0.0, buffer_size=4)
    cl.update("b1"), cl.update("b2")
    skill = iter([1.0, 0.99, 0.5])
    assert cl.prevent_forgetting(0.95, lambda: next(skill)) and cl.prevent_forgetting(0.95, lambda: next(skill))
    n = len(learn_log)
    assert not cl.prevent_forgetting(0.95, lambda: next(skill)) and len(learn_log) == n + 2        # the buffer was replayed
    kd = A.KnowledgeDistillation(2.0, 0.5)
    teacher, student = torch.nn.Linear(4, 3), torch.nn.Linear(4, 3)
    data = [(torch.randn(8, 4), torch.randint(0, 3, (8,))) for _ in range(30)]
    first = float(kd.loss(student(data[0][0]), teacher(data[0][0]).detach(), data[0][1]).detach())
    assert kd.distill(data, 30, student, teacher) < first
    po = A.PromptOptimizer(lambda p: float(len(p)))
    assert po.evaluate("abc", "de") == 5.0
    cot = A.ChainOfThought(lambda p: "therefore the answer is 4" if "Step" in p and "Final" not in p else "4")
    assert cot.reason("2+2?", 5) == "4" and cot.get_chain() == ["therefore the answer is 4"]
    tu = A.ToolUse()
    tu.register("upper", lambda s: s.upper())
    assert tu.call_tool("upper", "abc") == "ABC" and tu.call_tool("nope").startswith("error") and tu.get_available_tools() == ["upper"]
    ms = A.MemorySystem(short_capacity=4)
    ms.store("the cat sat on the mat"), ms.store("the cat sat on the mat!"), ms.store("kernels run on the gpu")
    ms.consolidate()
    assert len(ms.long) == 2 and ms.short == [] and ms.retrieve("gpu kernels", 1) == ["kernels run on the gpu"]
    ms.store(torch.tensor([1.0, 0.0]), "east"), ms.store(torch.tensor([0.0, 1.0]), "north")
    assert ms.retrieve(torch.tensor([0.9, 0.1]), 1) == ["east"]
    eh = A.EvaluationHarness(lambda p: "4" if "2+2" in p else "?")
    eh.register("tiny", [("2+2", "4"), ("3+3", "6")])
    assert eh.evaluate("tiny")["accuracy"] == 0.5 and [r["benchmark"] for r in eh.evaluate_all()] == ["tiny"]
    fw = A.Flywheel(eh, lambda failures: None)
    fw.run([("2+2", "4"), ("3+3", "6")], max_iterations=3)
    assert len(fw.get_history()) == 3 and fw.get_no_improvement_count() == 2 and fw.get_log_path() == ""
    assert fw.self_play_for_test().startswith("iteration 0: accuracy")
    cg = A.CodeGenSelfImprover()
    assert cg.generate_kernel("no_such_op", 4) == "" and not cg.compile_and_test("") and not cg.replace_kernel("x", "")
    ok_src = "__global__ void k(float* x) { x[threadIdx.x] += 1.0f; }\n"
    assert cg.compile_and_test(ok_src) and not cg.compile_and_test("__global__ void k( {") and cg.replace_kernel("inc", ok_src)
    assert cg.candidates["inc"] == ok_src
    assert hasattr(A.HPOptimizer(), "population_based_training") and hasattr(A.NeuralArchitectureSearch(), "search")
