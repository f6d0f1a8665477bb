"""Process-group tree description: named nodes with sizes; leaf sizes multiply up to their parents."""


class ProcessGroupNode:
    def __init__(self, name, size=None):
        self.name = name
        self.size = size

    def __repr__(self):
        return f"ProcessGroupNode(name={self.name}, size={self.size})"


class ProcessGroupConfig:
    def __init__(self, node):
        self.root = node
        self.root_id = node.name
        self.nodes = {node.name: node}
        self.children = {node.name: []}
        self.parent = {node.name: None}

    def add_node(self, node, parent=None):
        if parent is None:
            parent = self.root_id
        if isinstance(parent, ProcessGroupNode):
            parent = parent.name
        assert parent in self.nodes, f"unknown parent {parent}"
        self.nodes[node.name] = node
        self.children[node.name] = []
        self.children[parent].append(node.name)
        self.parent[node.name] = parent

    def get_node(self, name):
        return self.nodes[name]

    def leaf_groups(self):
        return [n for n, c in self.children.items() if not c]

    def set_leaf_group_sizes(self, group_sizes, update_parent_sizes=True):
        for name, size in group_sizes.items():
            assert not self.children[name], f"{name} is not a leaf group"
            self.nodes[name].size = size
        if update_parent_sizes:
            return self.update_parent_sizes()

    def update_parent_sizes(self, verbose=False):
        def fill(name):
            kids = self.children[name]
            if not kids:
                return self.nodes[name].size
            prod = 1
            for k in kids:
                prod *= fill(k)
            if name == self.root_id and self.nodes[name].size is not None:
                assert self.nodes[name].size == prod, f"group sizes multiply to {prod}, world has {self.nodes[name].size} ranks"
            self.nodes[name].size = prod
            return prod

        fill(self.root_id)
        return {n: v.size for n, v in self.nodes.items()}
