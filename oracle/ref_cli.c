/* Entry point of oracle/_ref/ggnpu_cpu_oracle: the reference CLI (its own
 * main(), renamed inside ref_shim.cpp) running on the reference CPU backend.
 * TEST INFRASTRUCTURE ONLY. */
int ref_cli_main(int argc, char** argv);
int main(int argc, char** argv) { return ref_cli_main(argc, argv); }
