"""Agentic layer: monitoring, safety, search, memory, planning, distillation, code generation and
the self-improvement flywheel (sandboxed g++ builds in a temp directory)."""
import json
import os
import shutil

import pytest
import torch
import torch.nn as nn

from mythos_b200.apps import asi


class ToyModel:
    """Deterministic text model: confident after the word 'sure', otherwise flat."""

    def generate_text(self, prompt, max_tokens=16):
        if "Step 1" in prompt and "Step 2" not in prompt:
            return "compute the sum"
        if "Step" in prompt:
            return "therefore the answer is 4"
        if "Numbered steps" in prompt:
            return "1. gather data\n2. train\n3. evaluate"
        return "2"

    def next_token_logits(self, text):
        lg = torch.zeros(50)
        if "sure" in text or "expert" in text:
            lg[3] = 12.0
        return lg


def test_monitor_reflection_and_prompt_search():
    m = ToyModel()
    assert asi.SelfMonitor.estimate_confidence(torch.zeros(10)) < 1e-6
    assert asi.SelfMonitor.estimate_confidence(torch.tensor([20.0, 0, 0, 0])) > 0.9
    st = asi.SelfMonitor(m).analyze("q", "a b c")
    assert st.needs_reanalysis and len(st.token_confidences) == 3
    assert asi.SelfMonitor(m).analyze("sure", "a").confidence > 0.5
    assert isinstance(asi.SelfReflector(m).refine("x", asi.SelfReflector(m).reflect("q", "x")), str)
    best = asi.PromptOptimizer(m, seed=1).optimize("task", 30)
    assert "expert" in best
    cot = asi.ChainOfThought(m)
    assert "answer" in cot.reason("2+2") and len(cot.get_chain()) == 2
    assert asi.CapabilityAmplifier(m).measure("arithmetic") < 0.1


def test_safety_alignment_hitl_tools():
    g = asi.SafetyGuardrails()
    assert g.check_input("hello") and not g.check_output("sudo rm -rf / now")
    g.set_kill_switch(True)
    assert g.is_killed() and not g.check_output("hello")
    h = asi.HITL()
    assert h.request_approval("deploy")
    h.pause()
    assert not h.request_approval("deploy") and h.is_paused()
    assert asi.HITL(approver=lambda a: a == "ok").request_approval("ok")
    al = asi.AlignmentSystem()
    assert al.value_alignment_score("happy to help, be careful") > al.value_alignment_score("attack and destroy")
    t = asi.ToolUse()
    assert t.call_tool("calculator", "2*(3+4)") == "14" and t.call_tool("calculator", "__import__('os')").startswith("error")
    assert t.call_tool("calculator", "9**9**9**9").startswith("error")          # no powers, no unbounded work
    assert t.call_tool("calculator", "-(7 % 4) + 10 / 4") == "-0.5" and t.call_tool("calculator", "1/0").startswith("error")
    assert t.call_tool("calculator", "+".join(["1"] * 100)).startswith("error")
    assert t.call_tool("nope", "") .startswith("error") and "upper" in t.get_available_tools()


def test_search_world_model_memory_planning():
    best = asi.NeuralArchitectureSearch(seed=0).search(20, 10)
    params = 12 * best.layers * best.hidden ** 2
    assert 1e8 < params < 1e9            # analytic optimum is at 1 / (2e-9 ln 10) ~ 2.2e8 parameters
    hp = asi.HPOptimizer(lambda c: -(c["lr"] - 0.3) ** 2, {"lr": (0.0, 1.0)}, seed=0).population_based_training(8, 12)
    assert abs(hp["lr"] - 0.3) < 0.1
    wm = asi.WorldModel(3, 2, seed=1)
    S, A = torch.randn(200, 3) * 0.5, torch.randn(200, 2) * 0.5
    S2 = torch.stack([wm.simulate_step(s, a) for s, a in zip(S, A)])
    fit = asi.WorldModel(3, 2, seed=5)
    fit.fit(S, A, S2)
    assert torch.allclose(fit.A, wm.A, atol=1e-3) and torch.allclose(fit.B, wm.B, atol=1e-3)
    assert len(wm.plan(torch.zeros(3), torch.ones(3) * 0.1, horizon=3, candidates=8)) == 3
    ex = asi.CuriosityDrivenExplorer(lambda s, a: s + torch.tensor([1.0, 0.0]) * (a - 0.5), 2)
    assert len(ex.explore(torch.zeros(2), 5)) == 5 and len(ex.visited) == 5
    mem = asi.MemorySystem(capacity=3)
    for i in range(4):
        mem.store(torch.eye(4)[i], f"v{i}")
    assert mem.retrieve(torch.eye(4)[2], k=1) == ["v2"] and len(mem.keys) == 3
    mem.store(torch.eye(4)[2] * 2, "dup")
    assert mem.consolidate() == 1
    plan = asi.PlanningEngine(ToyModel()).plan("ship it")
    assert [p.action for p in plan] == ["gather data", "train", "evaluate"] and asi.PlanningEngine().execute(plan)
    assert not asi.PlanningEngine().execute(list(reversed(plan)))
    mas = asi.MultiAgentSystem(3)
    mas.run_episode(2)
    assert all(len(h) >= 2 for h in mas.get_histories())
    res = asi.EvaluationHarness(ToyModel()).evaluate_all()
    assert res[0].accuracy == 0.5 and res[0].samples == 2
    cl = asi.ContinuousLearner(evaluate=lambda ex: 1.0, capacity=4)
    cl.update(range(10))
    assert len(cl.exemplars) == 4 and cl.prevent_forgetting()
    imp = asi.RecursiveSelfImprover(lambda c: -abs(c["hidden_size"] - 512), {"hidden_size": 256})
    assert imp.improvement_cycle(6)["hidden_size"] > 256


def test_distillation_updates_the_student():
    torch.manual_seed(0)
    teacher, student = nn.Linear(8, 5), nn.Linear(8, 5)
    kd = asi.KnowledgeDistillation(teacher, student, temperature=2.0, lr=5e-2)
    data = [torch.randn(16, 8) for _ in range(4)]
    losses = kd.distill(data, 60)
    assert losses[-1] < 0.3 * losses[0]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_codegen_and_flywheel(tmp_path):
    cg = asi.CodeGenSelfImprover(language="cpp")
    code = cg.generate_kernel("my gemm", 8, 8, 8)
    assert "gen_my_gemm" in code and cg.compile_and_test(code) and not cg.compile_and_test("int main( {")
    assert cg.replace_kernel("gemm", code) and "gemm" in cg.kernels
    cuda = asi.CodeGenSelfImprover(language="cuda").generate_kernel("g", 64, 64, 64)
    assert "__global__" in cuda
    v = asi.SelfVerifier()
    assert v.verify("p", "int f() { return (1); }") and not v.verify("p", "int f() { return (1; }")
    assert "division by zero" in v.find_edge_cases("a / b")
    fw = asi.Flywheel(workdir=str(tmp_path), patience=2)
    hist = fw.run(6)
    assert hist[0].compiled and hist[0].verified and hist[0].applied and os.path.exists(hist[0].file)
    assert hist[-1].delta <= 0 and fw.check_convergence()           # the same solutions stop improving
    lines = [json.loads(ln) for ln in open(fw.get_log_path())]
    assert len(lines) == len(hist) and lines[0]["task"] == "sum_array"
    bad = fw.sandbox_compile_and_test("int solve(const int* a, int n) { while (1) {} return 0; }", "CHECK(solve(0, 0) == 0);", 0.5)
    assert bad.compiled and not bad.passed
    assert fw.calculate_cyclomatic_complexity("if (a && b) for (;;) {}") == 4 and fw.measure_nesting_depth("{{}{}}") == 2
    assert "+b" in fw.make_diff("a\n", "b\n")
