"""Hand-built chains shared by simulator / planner / engine tests."""
from dataflow_b200.sim import Object, OutputAlloc, Task, TaskChain, TransferTrigger


def train_chain(L=8, rounds=2, W=400, O=800, A=300, Y=50, tf=100, tb=200, to=50, bw=4):
    """A training-shaped chain: L layers, fwd/bwd per round, interleaved optimizer in the last round."""
    init = [Object("tok", 10, "backing", "other")]
    for i in range(L):
        init += [Object(f"W{i}", W, "backing", "weight"), Object(f"O{i}", O, "backing", "optimizer")]
    tasks = []
    for r in range(rounds):
        prev = "tok"
        for i in range(L):
            tasks.append(Task(f"f{r}_{i}", [prev, f"W{i}"], [OutputAlloc(f"y{r}_{i}", Y), OutputAlloc(f"A{r}_{i}", A, "fast", "activation")], tf))
            prev = f"y{r}_{i}"
        dy = prev
        for i in reversed(range(L)):
            ins = [dy, f"A{r}_{i}", f"W{i}"]
            outs = [OutputAlloc(f"dy{r}_{i}", Y)]
            mut = []
            if r == 0:
                outs.append(OutputAlloc(f"dW{i}", W, "fast", "gradient"))
            else:
                ins.append(f"dW{i}")
                mut = [f"dW{i}"]
            tasks.append(Task(f"b{r}_{i}", ins, outs, tb, mutates_inputs=mut))
            dy = f"dy{r}_{i}"
            if r == rounds - 1:
                tasks.append(Task(f"o{i}", [f"W{i}", f"dW{i}", f"O{i}"], [], to, mutates_inputs=[f"W{i}", f"O{i}"]))
    fin = {f"W{i}": "backing" for i in range(L)}
    fin.update({f"O{i}": "backing" for i in range(L)})
    return TaskChain(init, tasks, fin, None, None, bw, bw)
