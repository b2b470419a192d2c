// Process-wide count of kernel launches issued by this library's launchers (a launch captured into a
// CUDA graph counts once, at capture).
#pragma once
extern "C" void eredu_count_launches(int n);
extern "C" long long eredu_launch_count();
