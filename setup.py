from setuptools import find_packages, setup

setup(
    name="allie-b200",
    version="0.1.0",
    description="Blackwell-native framework with the capabilities of y0mingzhang/allie",
    packages=find_packages(include=["allie_b200", "allie_b200.*"]) + ["modeling", "evaluation", "server", "data"],
    package_dir={"modeling": "src/modeling", "evaluation": "src/evaluation", "server": "src/server",
                 "data": "src/data"},
    package_data={"allie_b200": ["lib/*.so", "csrc/*", "serve/*.sh", "etl/*.sh"]},
    install_requires=["torch>=2.6", "numpy", "pyyaml"],
    extras_require={"hf": ["transformers"], "metrics": ["wandb"], "etl": ["zstandard"]},
    entry_points={"console_scripts": ["allie = allie_b200.__main__:main"]},
    python_requires=">=3.10",
)
